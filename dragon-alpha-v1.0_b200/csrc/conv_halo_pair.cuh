// Stride-1 forward conv / deltaX on CTA pairs (clusters of two, tcgen05 cta_group::2).
//
// Same tiling as conv_halo_kernel with one accumulator (16 x 8 pixels) per CTA, but two CTAs of a
// cluster work on neighbouring pixel tiles of the same output-channel block and share every MMA:
// the leader (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256, each CTA supplies the
// A rows of its own patch and HALF of the rows of the W tile from the same shared-memory offsets,
// and each CTA's tensor memory receives its own 128 rows of D.  A tcgen05.mma reads 4 KB of A plus
// 32 B per B row from shared memory, and an MMA of 128 columns already uses the whole 128 B/clk of
// one SM; splitting B over two SMs halves both those reads and the TMA writes of the W tiles.
//
// W tile of one tap in each CTA (K-major, 128-byte rows, BN = output channels of the block):
//   plain TF32:  rows [rank * BN/2, (rank+1) * BN/2) of W.                   N = BN
//   3xTF32:      the CTA's BN/2 rows of W_hi followed by its BN/2 rows of W_lo; three MMAs of N = BN,
//                with BN <= 128 the two correction terms into a second set of BN columns.
//   wide 3xTF32: region P (BN rows): all of W_hi in the leader, all of W_lo in the peer, so that
//                x_hi * [W_hi | W_lo] is one MMA of N = 2*BN; region Q (BN/2 rows): the CTA's half
//                of W_hi for x_lo * W_hi (N = BN), which accumulates in the second BN columns.
//
// Barriers the leader's MMA thread waits on (B full, patch full / ready, accumulator empty) live in
// the leader's shared memory; the peer's TMA loads count their bytes there and its warps arrive
// there through cluster addresses.  Barriers the other roles wait on (B empty, patch empty,
// accumulator full) exist in both CTAs and the leader commits to both.  Every wait is bounded.
//
// Warps per CTA: 0 TMA producer, 1 MMA issuer (leader only; both allocate tensor memory),
// 2-5 epilogue, 6-9 operand split.
#pragma once
#include "conv_halo.cuh"

namespace alpha {

template <int MODE, uint32_t kPW8>
__device__ __forceinline__ void issue_chunk_pair(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t a_lo_off, uint32_t q_off, uint32_t idesc, uint32_t idesc_wide,
                                                 uint32_t side_off, uint32_t acc_first)
{
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const uint32_t a_k = a_lo + kk * 2, b_k = b_lo + kk * 2;
        const uint32_t acc = kk == 0 ? acc_first : 1u;
        if (MODE == 2) {
            mma_tf32_pair(d, a_k, a_hi, b_k, b_hi, idesc_wide, acc);
            mma_tf32_pair(d + side_off, a_k + a_lo_off, a_hi, b_k + q_off, b_hi, idesc, 1u);
        } else if (MODE == 4) {
            // three products, the two correction terms into the side columns (see conv_halo.cuh: the
            // tensor core truncates when it accumulates, so only hi x hi goes into the main sum)
            mma_tf32_pair(d + side_off, a_k + a_lo_off, a_hi, b_k, b_hi, idesc, acc);
            mma_tf32_pair(d + side_off, a_k, a_hi, b_k + q_off, b_hi, idesc, 1u);
            mma_tf32_pair(d, a_k, a_hi, b_k, b_hi, idesc, acc);
        } else if (MODE == 1) {
            // three products into one accumulator; q_off = distance from this CTA's W_hi rows to its W_lo rows
            mma_tf32_pair(d, a_k + a_lo_off, a_hi, b_k, b_hi, idesc, acc);
            mma_tf32_pair(d, a_k, a_hi, b_k + q_off, b_hi, idesc, 1u);
            mma_tf32_pair(d, a_k, a_hi, b_k, b_hi, idesc, 1u);
        } else {
            mma_tf32_pair(d, a_k, a_hi, b_k, b_hi, idesc, acc);
        }
    }
}

// FW_T: compile-time filter width; ROW_T: one B stage holds the FW_T taps of a filter row.
// FLAT_T: the accumulator is 4 output rows x 32 patch columns instead of 16 x 8: the patch has a pitch of exactly 32
// pixels, so the 128 lanes are 128 CONSECUTIVE patch positions (8-row groups 1024 B apart), a tap is still a constant
// shift (fh * 32 + fw positions), and the columns 30, 31 of every row are idle lanes.  For images at most 30 pixels
// wide whose height 16 x 8 tiles fill badly (28 x 28: 0.875 of the lanes instead of 0.77); the epilogue's 32-column
// store box is clipped at the image edge by the TMA.
// p.mode3x is 0 (plain TF32), 1 (3xTF32, three MMAs), 4 (the same with side columns) or 2 (wide 3xTF32); p.JH == p.JW == 1; p.total_tiles is even and the
// tiles 2k, 2k+1 lie in the same output-channel block.  p.b_bytes = bytes of one tap's W tile per CTA.
template <int FW_T, bool ROW_T, bool FLAT_T = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kHaloThreads, 1)
    conv_halo_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmO,
                          const HaloParams p)
{
    constexpr int tps = ROW_T ? FW_T : 1;
    const int stages_per_chunk = ROW_T ? p.FH : p.FH * FW_T;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const bool wide = p.mode3x == 2, three = p.mode3x == 1 || p.mode3x == 4;
    const bool side = wide || p.mode3x == 4;   // accumulators are 2 * BN columns, the epilogue adds the halves
    const uint32_t planes = p.mode3x ? 2u : 1u;
    const uint32_t patch_stride = p.patch_bytes * planes;
    const uint32_t b_tile = p.b_bytes;             // one tap, this CTA's share
    const uint32_t b_stride = b_tile * tps;
    uint8_t* patches = smem;
    uint8_t* bring = smem + static_cast<size_t>(p.npb) * patch_stride;
    uint8_t* staging = bring + static_cast<size_t>(p.sb) * b_stride;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * 16384);
    uint64_t* patch_full = bars;
    uint64_t* patch_ready = patch_full + p.npb;
    uint64_t* patch_empty = patch_ready + p.npb;
    uint64_t* b_full = patch_empty + p.npb;
    uint64_t* b_empty = b_full + p.sb;
    uint64_t* acc_full = b_empty + p.sb;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.npb; ++i) {
            mbar_init(&patch_full[i], 1);
            mbar_init(&patch_ready[i], 256);   // the split warps of both CTAs
            mbar_init(&patch_empty[i], 1);
        }
        for (int i = 0; i < p.sb; ++i) {
            mbar_init(&b_full[i], 1);
            mbar_init(&b_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 256);     // the epilogue warps of both CTAs
        }
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        prefetch_tmap(&tmBlo);
        prefetch_tmap(&tmO);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_holder, p.tmem_cols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised before anything reaches them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int per_img = p.row_blocks * p.col_blocks;
    const int pair_tiles = p.total_tiles >> 1;
    const int n_pairs = gridDim.x >> 1, pair_id = blockIdx.x >> 1;

    const uint32_t patches_a = smem_u32(patches), bring_a = smem_u32(bring);
    const uint32_t pfull_a = smem_u32(patch_full), pready_a = smem_u32(patch_ready), pempty_a = smem_u32(patch_empty);
    const uint32_t bfull_a = smem_u32(b_full), bempty_a = smem_u32(b_empty);
    const uint32_t afull_a = smem_u32(acc_full), aempty_a = smem_u32(acc_empty);
    // the same barriers seen through the cluster window
    const uint32_t pfull_L = mapa_u32(pfull_a, 0), pready_L = mapa_u32(pready_a, 0);
    const uint32_t bfull_L = mapa_u32(bfull_a, 0), aempty_L = mapa_u32(aempty_a, 0);
    const uint32_t pempty_0 = mapa_u32(pempty_a, 0), pempty_1 = mapa_u32(pempty_a, 1);
    const uint32_t bempty_0 = mapa_u32(bempty_a, 0), bempty_1 = mapa_u32(bempty_a, 1);
    const uint32_t afull_0 = mapa_u32(afull_a, 0), afull_1 = mapa_u32(afull_a, 1);
    const uint32_t half_rows = static_cast<uint32_t>(p.BN) >> 1;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer (both CTAs) ----
            RingPos pp, bp;
            bool ok = true;
            const int taps = p.FH * FW_T;
            for (int pt = pair_id; pt < pair_tiles && ok; pt += n_pairs) {
                const int t = 2 * pt + static_cast<int>(rank);
                const int tn = t / (p.n_blocks * per_img);
                int r = t - tn * (p.n_blocks * per_img);
                const int nb = r / per_img;
                r -= nb * per_img;
                const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
                const int h0 = rb * (FLAT_T ? 4 : 16) - p.pad_h, w0 = FLAT_T ? -p.pad_w : cb * 8 - p.pad_w;
                const int n = nb * p.NI;
                const int oc0 = tn * p.BN;
                for (int c = 0; c < p.kchunks && ok; ++c) {
                    if (!mbar_wait_a(pempty_a + 8 * pp.idx, pp.phase ^ 1)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                    if (p.mode3x) {
                        // the split warps of this CTA wait for the patch: count it locally
                        mbar_arrive_expect_tx_a(pfull_a + 8 * pp.idx, p.patch_tx);
                        tma_load_4d_a(patches_a + pp.idx * patch_stride, &tmA, pfull_a + 8 * pp.idx, c * 32, w0, h0, n);
                    } else {
                        // the leader's MMA thread waits for both patches
                        if (leader) mbar_arrive_expect_tx_a(pfull_a + 8 * pp.idx, 2 * p.patch_tx);
                        tma_load_4d_pair(patches_a + pp.idx * patch_stride, &tmA, pfull_L + 8 * pp.idx, c * 32, w0, h0, n);
                    }
                    pp.advance(p.npb);
                    for (int st = 0; st < stages_per_chunk; ++st) {
                        if (!mbar_wait_a(bempty_a + 8 * bp.idx, bp.phase ^ 1)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                        if (leader) mbar_arrive_expect_tx_a(bfull_a + 8 * bp.idx, 2 * p.b_tx * tps);
                        const uint32_t bar = bfull_L + 8 * bp.idx;
                        for (int q = 0; q < tps; ++q) {
                            const int tap = st * tps + q;
                            const uint32_t b_dst = bring_a + bp.idx * b_stride + q * b_tile;
                            const int my_half = oc0 + static_cast<int>(rank * half_rows);
                            if (three) {
                                tma_load_3d_pair(b_dst, &tmB, bar, c * 32, tap, my_half);
                                tma_load_3d_pair(b_dst + half_rows * 128, &tmBlo, bar, c * 32, tap, my_half);
                            } else if (!wide) {
                                tma_load_3d_pair(b_dst, &tmB, bar, c * 32, tap, my_half);
                            } else {
                                // P: W_hi (leader) or W_lo (peer), both halves; Q: this CTA's half of W_hi
                                const CUtensorMap* mp = leader ? &tmB : &tmBlo;
                                tma_load_3d_pair(b_dst, mp, bar, c * 32, tap, oc0);
                                tma_load_3d_pair(b_dst + half_rows * 128, mp, bar, c * 32, tap, oc0 + static_cast<int>(half_rows));
                                tma_load_3d_pair(b_dst + 2 * half_rows * 128, &tmB, bar, c * 32, tap, my_half);
                            }
                        }
                        bp.advance(p.sb);
                    }
                }
            }
            (void)taps;
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---- MMA issuer (leader CTA only) ----
            RingPos pp, bp, ap;
            bool ok = true;
            constexpr uint32_t kPW8 = FLAT_T ? 256u : (8 + FW_T - 1) * 8;   // one patch row, in 16-byte units
            const uint32_t a_dhi = smem_desc_hi(FLAT_T ? 1024u : p.PW * 128, kSwizzle128B);
            const uint32_t b_dhi = smem_desc_hi(1024, kSwizzle128B);
            const uint32_t a_lo_off = p.patch_bytes >> 4;
            const uint32_t q_off = ((three ? 1u : 2u) * half_rows * 128) >> 4;   // region Q of a wide W tile / the W_lo rows
            const uint32_t patch_lo0 = smem_desc_lo(patches_a, 16), patch_stride16 = patch_stride >> 4;
            const uint32_t bring_lo0 = smem_desc_lo(bring_a, 16), b_stride16 = b_stride >> 4, b_tile16 = b_tile >> 4;
            const uint32_t pwait_a = p.mode3x ? pready_a : pfull_a;
            const uint32_t accw = side ? 2u * p.BN : p.BN;
            const bool prof_on = p.prof != nullptr && blockIdx.x == 0;
            unsigned long long w_patch = 0, w_b = 0, w_acc = 0;
            const long long t_begin = clock64();
            auto timed_wait = [&](uint32_t bar, uint32_t parity, unsigned long long& acc) {
                if (!prof_on) return mbar_wait_cluster_a(bar, parity);
                const long long t0 = clock64();
                const bool r = mbar_wait_cluster_a(bar, parity);
                acc += static_cast<unsigned long long>(clock64() - t0);
                return r;
            };
            for (int pt = pair_id; pt < pair_tiles && ok; pt += n_pairs) {
                if (!timed_wait(aempty_a + 8 * ap.idx, ap.phase ^ 1, w_acc)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d0 = tmem_base + ap.idx * accw;
                uint32_t acc_first = 0u;
                for (int c = 0; c < p.kchunks && ok; ++c) {
                    if (!timed_wait(pwait_a + 8 * pp.idx, pp.phase, w_patch)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after_sync();
                    uint32_t a_row = patch_lo0 + pp.idx * patch_stride16;
                    for (int fh = 0; fh < p.FH && ok; ++fh, a_row += kPW8) {
                        if (ROW_T) {
                            if (!timed_wait(bfull_a + 8 * bp.idx, bp.phase, w_b)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                            tc_fence_after_sync();
                            const uint32_t bl = bring_lo0 + bp.idx * b_stride16;
                            if (wide) {
#pragma unroll
                                for (int fw = 0; fw < FW_T; ++fw)
                                    issue_chunk_pair<2, kPW8>(d0, a_row + fw * 8, a_dhi, bl + fw * b_tile16, b_dhi, a_lo_off, q_off,
                                                              p.idesc, p.idesc_wide, p.BN, fw == 0 ? acc_first : 1u);
                            } else if (p.mode3x == 4) {
#pragma unroll
                                for (int fw = 0; fw < FW_T; ++fw)
                                    issue_chunk_pair<4, kPW8>(d0, a_row + fw * 8, a_dhi, bl + fw * b_tile16, b_dhi, a_lo_off, q_off,
                                                              p.idesc, p.idesc_wide, p.BN, fw == 0 ? acc_first : 1u);
                            } else if (three) {
#pragma unroll
                                for (int fw = 0; fw < FW_T; ++fw)
                                    issue_chunk_pair<1, kPW8>(d0, a_row + fw * 8, a_dhi, bl + fw * b_tile16, b_dhi, a_lo_off, q_off,
                                                              p.idesc, p.idesc_wide, p.BN, fw == 0 ? acc_first : 1u);
                            } else {
#pragma unroll
                                for (int fw = 0; fw < FW_T; ++fw)
                                    issue_chunk_pair<0, kPW8>(d0, a_row + fw * 8, a_dhi, bl + fw * b_tile16, b_dhi, a_lo_off, q_off,
                                                              p.idesc, p.idesc_wide, p.BN, fw == 0 ? acc_first : 1u);
                            }
                            acc_first = 1u;
                            mma_commit_pair(bempty_0 + 8 * bp.idx);
                            mma_commit_pair(bempty_1 + 8 * bp.idx);
                            bp.advance(p.sb);
                        } else {
#pragma unroll
                            for (int fw = 0; fw < FW_T; ++fw) {
                                if (!timed_wait(bfull_a + 8 * bp.idx, bp.phase, w_b)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                                tc_fence_after_sync();
                                const uint32_t bl = bring_lo0 + bp.idx * b_stride16;
                                if (wide)
                                    issue_chunk_pair<2, kPW8>(d0, a_row + fw * 8, a_dhi, bl, b_dhi, a_lo_off, q_off, p.idesc,
                                                              p.idesc_wide, p.BN, acc_first);
                                else if (p.mode3x == 4)
                                    issue_chunk_pair<4, kPW8>(d0, a_row + fw * 8, a_dhi, bl, b_dhi, a_lo_off, q_off, p.idesc,
                                                              p.idesc_wide, p.BN, acc_first);
                                else if (three)
                                    issue_chunk_pair<1, kPW8>(d0, a_row + fw * 8, a_dhi, bl, b_dhi, a_lo_off, q_off, p.idesc,
                                                              p.idesc_wide, p.BN, acc_first);
                                else
                                    issue_chunk_pair<0, kPW8>(d0, a_row + fw * 8, a_dhi, bl, b_dhi, a_lo_off, q_off, p.idesc,
                                                              p.idesc_wide, p.BN, acc_first);
                                acc_first = 1u;
                                mma_commit_pair(bempty_0 + 8 * bp.idx);
                                mma_commit_pair(bempty_1 + 8 * bp.idx);
                                bp.advance(p.sb);
                            }
                        }
                    }
                    mma_commit_pair(pempty_0 + 8 * pp.idx);
                    mma_commit_pair(pempty_1 + 8 * pp.idx);
                    pp.advance(p.npb);
                }
                mma_commit_pair(afull_0 + 8 * ap.idx);
                mma_commit_pair(afull_1 + 8 * ap.idx);
                ap.advance(p.acc_bufs);
            }
            if (prof_on) {
                p.prof[kProfMmaPatchWait] = w_patch; p.prof[kProfMmaBWait] = w_b; p.prof[kProfMmaAccWait] = w_acc;
                p.prof[kProfMmaTotal] = static_cast<unsigned long long>(clock64() - t_begin);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---- epilogue (both CTAs): warps 2..5, lane quadrant = warp % 4 ----
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        RingPos ap;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const uint32_t stage_a = smem_u32(staging);
        uint32_t sbuf = 0;
        const uint32_t accw = side ? 2u * p.BN : p.BN;
        for (int pt = pair_id; pt < pair_tiles; pt += n_pairs) {
            if (!mbar_wait_a(afull_a + 8 * ap.idx, ap.phase)) { report(p.status, kStatusEpilogueTimeout); break; }
            tc_fence_after_sync();
            const int t = 2 * pt + static_cast<int>(rank);
            const int tn = t / (p.n_blocks * per_img);
            int r = t - tn * (p.n_blocks * per_img);
            const int nb = r / per_img;
            r -= nb * per_img;
            const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
            const int n = nb * p.NI;
            const int n0 = tn * p.BN;
            const int oh0 = rb * (FLAT_T ? 4 : 16), ow0 = FLAT_T ? 0 : cb * 8;
            const uint32_t tcol = lane_base + ap.idx * accw;
            for (int c = 0; c < p.BN; c += 32) {
                const int col0 = n0 + c;
                if (col0 >= p.Ncols) break;
                if (threadIdx.x == 64) tma_store_wait_read<1>();
                named_barrier_sync(1, 128);
                uint32_t v[32];
                tmem_ld_32x32(tcol + c, v);
                tmem_ld_wait();
                if (side) {
                    uint32_t w[32];
                    tmem_ld_32x32(tcol + p.BN + c, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 32; ++q) v[q] = __float_as_uint(__uint_as_float(v[q]) + __uint_as_float(w[q]));
                }
                const uint32_t srow = stage_a + sbuf * 16384 + row * 128;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float4 o = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                           __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                    if (p.bias && col0 + 4 * q < p.Ncols) {
                        const float4 b = *reinterpret_cast<const float4*>(p.bias + col0 + 4 * q);
                        o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                    }
                    if (p.act_on) leaky_relu4(o, p.act_k);
                    st_shared_v4(srow + ((q ^ (row & 7)) << 4), o);
                }
                fence_proxy_async_smem();
                named_barrier_sync(1, 128);
                if (threadIdx.x == 64) {
                    if (p.NI == 1) {
                        tma_store_4d_a(&tmO, stage_a + sbuf * 16384, col0, ow0, oh0, n);
                    } else {
                        for (int img = 0; img < p.NI; ++img)
                            if (n + img < p.N)
                                tma_store_4d_a(&tmO, stage_a + sbuf * 16384 + img * p.SG * 1024, col0, ow0, 0, n + img);
                    }
                    tma_store_commit();
                }
                sbuf ^= 1u;
            }
            tc_fence_before_sync();
            mbar_arrive_cluster(aempty_L + 8 * ap.idx);
            ap.advance(p.acc_bufs);
        }
        if (threadIdx.x == 64) tma_store_wait_all();
    } else {
        // ---- operand split (3xTF32, both CTAs): warps 6..9 ----
        if (p.mode3x) {
            const int tid128 = threadIdx.x - 192;
            RingPos pp;
            bool ok = true;
            for (int pt = pair_id; pt < pair_tiles && ok; pt += n_pairs) {
                for (int c = 0; c < p.kchunks && ok; ++c) {
                    if (!mbar_wait_a(pfull_a + 8 * pp.idx, pp.phase)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                    uint8_t* ph = patches + static_cast<size_t>(pp.idx) * patch_stride;
                    split_plane_lo_x4(ph, ph + p.patch_bytes, p.patch_tx, tid128, 128);
                    fence_proxy_async_smem();
                    mbar_arrive_cluster(pready_L + 8 * pp.idx);
                    pp.advance(p.npb);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves while the other may still reach its shared memory
    if (warp == 1) tmem_dealloc_pair(tmem_base, p.tmem_cols);
}

}  // namespace alpha
