// Stride-1 deltaW with each X and deltaY tile fetched once per filter row.
//
//   deltaW[oc][fh][fw][ic] = sum over pixels of deltaY[pix][oc] * X[pix shifted by (fh, fw)][ic]
//
// The reduction axis of this GEMM is the pixel axis, so both operands are MN-major in shared
// memory: a tile row is one pixel, its 128 bytes are 32 channels.  One tcgen05.mma (K = 8) consumes
// 8 consecutive pixels of one image row.  A CTA owns one accumulator group - one filter row fh
// (FW taps), one block of up to 128 output channels (M) and one block of NT input channels (N) -
// and a share of the pixel tiles.  For every pixel tile of R rows x CW columns it loads the
// deltaY tile and the X tile (R rows x (CW + FW - 1) columns, shifted by fh) once; the FW taps of
// the row are formed by starting the X descriptor fw pixel rows later (tensor cores apply the
// shared-memory swizzle to absolute addresses, so any 128-byte row is a valid start).  The CTA
// accumulates over all its pixel tiles in tensor memory and writes one partial per CTA at the end;
// dw_reduce_kernel sums the partials in a fixed order.
//
// 3xTF32 has two forms.  mode3x == 1: three MMAs per step (lo*hi, hi*lo, hi*hi) into one
// accumulator.  mode3x == 2 ("stacked"), for blocks of at most 64 output and 64 input channels,
// where an MMA costs the same as one twice as tall and twice as wide: the lo plane of deltaY is
// stacked under its hi plane (M = 64 + 64) and the lo plane of X beside its hi plane (N = NT + NT),
// so that ONE MMA forms all four products; the epilogue writes the hi rows (hi*hi + hi*lo) and the
// lo rows (lo*hi + lo*lo) as two partials and the reduction adds them.
//
// mode3x == 3 ("diagonal", plain TF32 with at most 64 output channels) uses the same stacked layout
// for two halves of the pixel tile instead of two precision planes: rows 0..R-1 and R..2R-1 of the
// tile land where the hi and lo planes would, one MMA multiplies [dY_a; dY_b] by [X_a | X_b], the
// diagonal quadrants dY_a*X_a and dY_b*X_b are the two partials and the off-diagonal ones are
// ignored - twice the pixels per MMA where the 128-row operand would be half empty.
//
// Bias gradient (p.bias_out): deltaB[oc] = sum over pixels of deltaY[pix][oc] needs exactly the tiles the
// groups with fh == 0, ict == 0 (and the first tap group) already stage.  Their split threads add up the fp32 words of every
// deltaY tile (thread t always meets the same four channels of a 32-channel block: its 16-byte chunk of the
// 128-byte pixel row and, with the 32-byte-atom swizzle, the row index modulo 4 do not change while it
// strides over 32 rows at a time), and after the loop the 32 threads of each channel quad are added in
// thread order.  Pixels outside the image and channels beyond OC arrive as zeros from the TMA.
//
// Strides 1 and 2.  With a stride the X pixels one tap meets lie sw columns (sh rows) apart, so X is addressed
// through one tensor map per phase of that lattice - rows (fh - ph) mod sh, fixed for a CTA, and columns
// (fw - pw) mod sw - whose tiles are dense again: a pixel tile stages one X tile per column phase its taps use
// (two for 3x3 and 4x4 stride 2, one for 1x1), and a tap starts its descriptor at its phase's tile plus
// floor((fw - pw) / sw) pixels.  Stride 1 is the case of one phase and a start of fw pixels.
//
// Filter rows of more than three taps (5x5, 7x7) at stride 1 may be split over several CTAs of G = 3 taps each, so
// that three accumulators of 128 columns fit tensor memory where five or seven would have to be 64 wide: tap group tg
// stages the X tile that starts G * tg columns further right; a last group with fewer taps runs its spare
// accumulator on the tile's last tap and never stores it.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2-9 operand split (3xTF32) during the loop, 2-5 epilogue after.
#pragma once
#include "conv_halo.cuh"

namespace alpha {

constexpr int kDwHaloThreads = 320;   // warp 0 TMA, 1 MMA, 2-9 operand split (3xTF32), 2-5 also epilogue
constexpr int kDwSplitThreads = 256;

struct DwHaloParams {
    float* out;            // partials [parts][OC][FH*FW][IC] (or deltaW itself when parts == 1)
    size_t part_stride;    // floats between two partials
    int* status;
    unsigned long long* prof;  // optional cycle counters of CTA (0,0): slots 0 producer wait, 2 MMA wait,
                               // 5 MMA total, 8 split wait, 9 split work, 10 kernel total
    int N, OH, OW;         // deltaY geometry
    int IC, OC, FH, FW, ph, pw;
    int NT;                // input channels per CTA (multiple of 32, <= 256)
    int ic_tiles, oc_tiles;  // IC / NT, ceil(OC / 128)
    int R, CW;             // pixel tile: rows x columns (CW multiple of 8)
    int PW;                // X tile columns = CW + FW - 1
    int row_blocks, col_blocks, tiles_per_img;
    int total_tiles;       // N * tiles_per_img
    int parts;             // CTAs per accumulator group = gridDim.x
    int per_image;         // 1: part i sums exactly the tiles of image i (parts == N) and `out` receives N separate results
    int stages, mode3x;    // mode3x: 0 plain TF32, 1 three MMAs, 2 stacked planes, 3 diagonal (TF32, two half tiles)
    uint32_t idesc, tmem_cols;
    uint32_t dy_blk, x_blk;   // bytes of one 32-channel block of the deltaY / X tile (multiples of 1024)
    uint32_t dy_tx, x_tx;     // bytes one block load delivers
    // Bias gradient fused into the pass over deltaY: when set, the CTAs of the accumulator groups with
    // fh == 0 and ict == 0 (one group per output-channel tile) also sum the columns of the deltaY tiles
    // they stage; CTA x of such a group writes its partial sums to bias_out[x * OC + oc].
    float* bias_out;
    // strided convolutions (see above): one X tile per column phase; all zero / one phase for stride 1
    int sh, sw;               // strides, 1 or 2
    int nph;                  // column phases staged per pixel tile (1 or 2)
    int G, tgroups;           // taps (accumulators) per CTA and CTAs per filter row: G = FW, tgroups = 1 unless a row of more
                              // than three taps is split (stride 1 only); the last group may own fewer than G real taps
    int col_q0[4];            // first lattice column of the X tile, relative to the tile's first output column: by column
                              // phase k (tgroups == 1) or by tap group (tgroups > 1, one phase)
    uint32_t tap_off16[8];    // start of tap fw's X tile within the X region of a stage, in 16-byte units
};

// X tensor maps by [row phase][column phase]; stride 1 uses entry 0
struct DwXMaps {
    CUtensorMap m[4];
};

// The MMAs of one staged pixel tile as straight-line code: all steps of one tap back to back.
// MODE 1 issues lo*hi, hi*lo, hi*hi per step; MODE 0 one MMA (plain TF32, or stacked planes).
template <int MODE, int FW_T, int R_T, int CW_T, bool STR_T>
__device__ __forceinline__ void dw_issue_tile(uint32_t tmem_base, uint32_t acc_cols, uint32_t a_s, uint32_t b_s,
                                              uint32_t lo_off, uint32_t dhi, uint32_t idesc, uint32_t acc,
                                              const uint32_t* __restrict__ toff)
{
    constexpr int kPW = CW_T + FW_T - 1;
#pragma unroll
    for (int fw = 0; fw < FW_T; ++fw) {
        const uint32_t d = tmem_base + fw * acc_cols;
#pragma unroll
        for (int r = 0; r < R_T; ++r)
#pragma unroll
            for (int g = 0; g < CW_T / 8; ++g) {
                const uint32_t a_k = a_s + (r * CW_T + g * 8) * 8;
                const uint32_t b_k = b_s + (STR_T ? toff[fw] : fw * 8) + (r * kPW + g * 8) * 8;
                const uint32_t first = (r | g) ? 1u : acc;
                if (MODE == 1) {
                    mma_tf32_ss2(d, a_k + lo_off, dhi, b_k, dhi, idesc, first);
                    mma_tf32_ss2(d, a_k, dhi, b_k + lo_off, dhi, idesc, 1u);
                    mma_tf32_ss2(d, a_k, dhi, b_k, dhi, idesc, 1u);
                } else {
                    mma_tf32_ss2(d, a_k, dhi, b_k, dhi, idesc, first);
                }
            }
    }
}

// The same with run-time filter width and tile shape (any filter); the math mode stays a template
// parameter so that no branch sits between two MMAs.
template <int MODE>
__device__ __forceinline__ void dw_issue_tile_rt(uint32_t tmem_base, uint32_t acc_cols, uint32_t a_s, uint32_t b_s, uint32_t lo_off,
                                                 uint32_t dhi, uint32_t idesc, uint32_t acc, int FW, int R, int CW, int PW,
                                                 const uint32_t* __restrict__ toff)
{
    uint32_t d = tmem_base;
    for (int fw = 0; fw < FW; ++fw, d += acc_cols) {
        uint32_t a_row = a_s, b_row = b_s + toff[fw];
        uint32_t first = acc;
        for (int r = 0; r < R; ++r, a_row += CW * 8, b_row += PW * 8) {
            uint32_t a_k = a_row, b_k = b_row;
            for (int g = 0; g < CW / 8; ++g, a_k += 64, b_k += 64) {
                if (MODE == 1) {
                    mma_tf32_ss2(d, a_k + lo_off, dhi, b_k, dhi, idesc, first);
                    mma_tf32_ss2(d, a_k, dhi, b_k + lo_off, dhi, idesc, 1u);
                    mma_tf32_ss2(d, a_k, dhi, b_k, dhi, idesc, 1u);
                } else {
                    mma_tf32_ss2(d, a_k, dhi, b_k, dhi, idesc, first);
                }
                first = 1u;
            }
        }
    }
}

// FW_T > 0: FW, R and CW are compile-time and the MMAs of a stage are straight-line code.
template <int FW_T, int R_T, int CW_T, bool STR_T = false>
__global__ void __launch_bounds__(kDwHaloThreads, 1)
    conv_dw_halo_kernel(const __grid_constant__ DwXMaps tmXs, const __grid_constant__ CUtensorMap tmDY,
                        const __grid_constant__ DwHaloParams p)
{
    constexpr bool kStatic = FW_T > 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.stages;
    const uint32_t planes = p.mode3x ? 2u : 1u;
    const int xb = p.NT / 32;                       // X blocks per stage
    const bool diag = p.mode3x == 3;
    const bool stacked = p.mode3x == 2 || diag;   // layout [dY a][dY b] [X a][X b], M = 64 + 64, N = NT + NT
    const int dyb = stacked ? 2 : 4;                // deltaY blocks per plane: 64 or 128 output channels
    const uint32_t dy_bytes = dyb * p.dy_blk;
    const uint32_t xph = xb * p.x_blk;             // X tile of one column phase
    const uint32_t x_bytes = p.nph * xph;
    const uint32_t plane_bytes = dy_bytes + x_bytes;
    const uint32_t stage_bytes = plane_bytes * planes;
    // stage layout.  modes 0/1: [dY hi][X hi] [dY lo][X lo];  mode 2: [dY hi][dY lo] then per column phase [X hi][X lo]
    const uint32_t x_off = stacked ? 2 * dy_bytes : dy_bytes;
    const uint32_t xph_stride = stacked ? 2 * xph : xph;   // between the tiles of two column phases
    const int oc_tile = stacked ? 64 : 128;
    const uint32_t acc_cols = stacked ? 2 * p.NT : p.NT;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S) * stage_bytes);
    uint64_t* full = bars;
    uint64_t* ready = bars + S;
    uint64_t* empty = bars + 2 * S;
    uint64_t* accum = bars + 3 * S;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 3 * S + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&ready[s], kDwSplitThreads);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        fence_barrier_init();
        prefetch_tmap(&tmXs.m[0]);
        prefetch_tmap(&tmDY);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    // accumulator group of this CTA
    const int grp0 = blockIdx.y;
    const int tg = grp0 % p.tgroups;          // tap group within the filter row
    const int grp = grp0 / p.tgroups;
    const int fw_base = tg * p.G;
    const int fh = grp % p.FH;
    const int ict = (grp / p.FH) % p.ic_tiles;
    const int oct = grp / (p.FH * p.ic_tiles);
    const int ic0 = ict * p.NT, oc0 = oct * oc_tile;
    // X rows of this filter row: lattice row qrow + (output row) of row phase phi
    const int drow = fh - p.ph;
    const int qrow = drow >= 0 ? drow / p.sh : -((-drow + p.sh - 1) / p.sh);
    const int phi = drow - qrow * p.sh;

    const uint32_t smem_a = smem_u32(smem);
    const uint32_t full_a = smem_u32(full), ready_a = smem_u32(ready), empty_a = smem_u32(empty);
    const int FW = kStatic ? FW_T : p.G;      // accumulators of this CTA
    const int R = kStatic ? R_T : p.R;
    const int CW = kStatic ? CW_T : p.CW;
    const int PW = CW + FW - 1;
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    // tiles of this CTA: every gridDim.x-th one, or (per_image) exactly the tiles of image blockIdx.x, whose sum
    // then is that image's own result (batched matrix products) and goes straight to the output
    const int t_first = p.per_image ? static_cast<int>(blockIdx.x) * p.tiles_per_img : static_cast<int>(blockIdx.x);
    const int t_last = p.per_image ? t_first + p.tiles_per_img : p.total_tiles;
    const int t_step = p.per_image ? 1 : static_cast<int>(gridDim.x);
    const long long t_kernel = clock64();
    const unsigned long long ns_kernel = prof_on ? globaltimer_ns() : 0ull;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            RingPos rp;
            unsigned long long w_empty = 0;
            for (int t = t_first; t < t_last; t += t_step) {
                const int n = t / p.tiles_per_img;
                const int r = t - n * p.tiles_per_img;
                const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
                if (!wait_prof(empty_a + 8 * rp.idx, rp.phase ^ 1, prof_on, w_empty)) { report(p.status, kStatusProducerTimeout); break; }
                const uint32_t bar = full_a + 8 * rp.idx;
                const uint32_t dst = smem_a + rp.idx * stage_bytes;
                const int halves = diag ? 2 : 1;
                mbar_arrive_expect_tx_a(bar, halves * (dyb * p.dy_tx + p.nph * xb * p.x_tx));
                const int ow0 = cb * CW;
                for (int h = 0; h < halves; ++h) {
                    const int oh0 = (rb * halves + h) * R;   // diagonal: the tile is 2R rows, one half per slot
                    for (int b = 0; b < dyb; ++b)
                        tma_load_4d_a(dst + h * dy_bytes + b * p.dy_blk, &tmDY, bar, oc0 + b * 32, ow0, oh0, n);
                    for (int k = 0; k < p.nph; ++k)
                        for (int b = 0; b < xb; ++b)
                            tma_load_4d_a(dst + x_off + k * xph_stride + h * xph + b * p.x_blk, &tmXs.m[phi * p.nph + k], bar,
                                          ic0 + b * 32, ow0 + p.col_q0[tg * p.nph + k], oh0 + qrow, n);
                }
                rp.advance(S);
            }
            if (prof_on) p.prof[kProfProducerPatchWait] = w_empty;
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            RingPos rp;
            const uint32_t dhi = smem_desc_hi(512, kSwizzle128B_Base32B);
            // a CTA that sums bias columns releases a stage only after its split threads have read it
            const bool do_bias = p.bias_out != nullptr && fh == 0 && ict == 0 && tg == 0;
            const uint32_t wait_a = (p.mode3x == 1 || p.mode3x == 2 || do_bias) ? ready_a : full_a;
            const bool three = p.mode3x == 1;
            const uint32_t stage16 = stage_bytes >> 4, lo_off = plane_bytes >> 4;
            const uint32_t a_lo0 = smem_desc_lo(smem_a, p.dy_blk);              // LBO = block stride
            const uint32_t b_lo0 = smem_desc_lo(smem_a + x_off, p.x_blk);
            uint32_t acc = 0u;  // the first MMA into each accumulator overwrites it
            unsigned long long w_in = 0, w_issue = 0, w_commit = 0;
            const long long t_begin = clock64();
            for (int t = t_first; t < t_last; t += t_step) {
                if (!wait_prof(wait_a + 8 * rp.idx, rp.phase, prof_on, w_in)) { report(p.status, kStatusMmaTimeout); break; }
                tc_fence_after_sync();
                const long long t_i0 = prof_on ? clock64() : 0;
                const uint32_t a_s = a_lo0 + rp.idx * stage16, b_s = b_lo0 + rp.idx * stage16;
                if constexpr (kStatic) {
                    // the mode test stays outside the unrolled MMAs: a branch per MMA costs the issuing
                    // thread more than the MMA takes
                    if (three) dw_issue_tile<1, FW_T, R_T, CW_T, STR_T>(tmem_base, acc_cols, a_s, b_s, lo_off, dhi, p.idesc, acc, p.tap_off16);
                    else dw_issue_tile<0, FW_T, R_T, CW_T, STR_T>(tmem_base, acc_cols, a_s, b_s, lo_off, dhi, p.idesc, acc, p.tap_off16);
                } else {
                    if (three) dw_issue_tile_rt<1>(tmem_base, acc_cols, a_s, b_s, lo_off, dhi, p.idesc, acc, FW, R, CW, PW, p.tap_off16);
                    else dw_issue_tile_rt<0>(tmem_base, acc_cols, a_s, b_s, lo_off, dhi, p.idesc, acc, FW, R, CW, PW, p.tap_off16);
                }
                acc = 1u;
                const long long t_i1 = prof_on ? clock64() : 0;
                mma_commit_a(empty_a + 8 * rp.idx);
                rp.advance(S);
                if (prof_on) { w_issue += t_i1 - t_i0; w_commit += clock64() - t_i1; }
            }
            mma_commit(accum);
            if (prof_on) {
                p.prof[kProfMmaPatchWait] = w_in; p.prof[kProfMmaBWait] = w_issue; p.prof[kProfMmaAccWait] = w_commit;
                p.prof[kProfMmaTotal] = static_cast<unsigned long long>(clock64() - t_begin);
            }
        }
        __syncwarp();
    } else {
        // ---- operand split while the loop runs (3xTF32): warps 2..9; epilogue afterwards: warps 2..5 ----
        const int tid128 = threadIdx.x - 64;   // index among the split threads
        bool ok = true;
        const bool split_on = p.mode3x == 1 || p.mode3x == 2;
        const bool do_bias = p.bias_out != nullptr && fh == 0 && ict == 0 && tg == 0;
        float4 bsum[4] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f),
                          make_float4(0.f, 0.f, 0.f, 0.f)};
        if (split_on || do_bias) {
            RingPos rp;
            unsigned long long w_full = 0;
            const long long t_begin = clock64();
            const int halves = diag ? 2 : 1;
            for (int t = t_first; t < t_last; t += t_step) {
                if (!wait_prof(full_a + 8 * rp.idx, rp.phase, prof_on, w_full)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                uint8_t* hi = smem + static_cast<size_t>(rp.idx) * stage_bytes;
                if (do_bias) {
                    // the staged fp32 words of deltaY (the split below leaves them as they are)
                    for (int h = 0; h < halves; ++h)
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            if (b >= dyb) break;
                            const uint8_t* blk = hi + h * dy_bytes + b * p.dy_blk;
                            for (uint32_t off = static_cast<uint32_t>(tid128) * 16u; off < p.dy_tx; off += kDwSplitThreads * 16u) {
                                const float4 v = *reinterpret_cast<const float4*>(blk + off);
                                bsum[b].x += v.x; bsum[b].y += v.y; bsum[b].z += v.z; bsum[b].w += v.w;
                            }
                        }
                }
                if (split_on) {
                    if (stacked) {
                        split_plane_lo_x4(hi, hi + dy_bytes, dy_bytes, tid128, kDwSplitThreads);
                        for (int k = 0; k < p.nph; ++k)
                            split_plane_lo_x4(hi + x_off + k * xph_stride, hi + x_off + k * xph_stride + xph, xph, tid128, kDwSplitThreads);
                    } else {
                        split_plane_lo_x4(hi, hi + plane_bytes, plane_bytes, tid128, kDwSplitThreads);
                    }
                    fence_proxy_async_smem();
                }
                mbar_arrive_a(ready_a + 8 * rp.idx);
                rp.advance(S);
            }
            if (prof_on && tid128 == 0) {
                p.prof[kProfSplitWait] = w_full;
                p.prof[kProfSplitWork] = static_cast<unsigned long long>(clock64() - t_begin) - w_full;
            }
        }
        if (do_bias) {
            // all MMAs have finished reading shared memory once `accum` completes; the ring then serves as
            // scratch for the cross-thread sum.  Every split thread takes part in the barrier, also one
            // whose wait ran out (the CTA then reports through the status word and its sums are void).
            const bool done = ok && mbar_wait(accum, 0);
            if (ok && !done) { report(p.status, kStatusEpilogueTimeout); ok = false; }
            float4* sc = reinterpret_cast<float4*>(smem);
#pragma unroll
            for (int b = 0; b < 4; ++b) sc[b * kDwSplitThreads + tid128] = bsum[b];
            named_barrier_sync(2, kDwSplitThreads);
            if (tid128 < dyb * 8) {
                const int b = tid128 >> 3, q = tid128 & 7;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int t = 0; t < kDwSplitThreads; ++t) {
                    // thread t reads 16-byte chunk (t & 7) of rows whose index modulo 4 is (t >> 3) & 3; the swizzle
                    // exchanges the 32-byte atoms of a row by that row index
                    const int quad = ((((t & 7) >> 1) ^ ((t >> 3) & 3)) << 1) | (t & 1);
                    if (quad == q) {
                        const float4 v = sc[b * kDwSplitThreads + t];
                        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                    }
                }
                const int oc = oc0 + b * 32 + q * 4;
                if (oc < p.OC) *reinterpret_cast<float4*>(p.bias_out + static_cast<size_t>(blockIdx.x) * p.OC + oc) = a;
            }
        }
        if (warp >= 6) ok = false;   // the extra split warps take no part in the epilogue
        if (ok && !mbar_wait(accum, 0)) { report(p.status, kStatusEpilogueTimeout); ok = false; }
        tc_fence_after_sync();
        if (ok) {
            const int quad = warp & 3;
            // stacked: tensor-memory lanes 0-63 are the hi rows, 64-127 the lo rows of the same channels
            const int oc = oc0 + (stacked ? (quad & 1) * 32 : quad * 32) + lane;
            const int sub = stacked ? (quad >> 1) : 0;
            const int nsub = stacked ? 2 : 1;
            const int taps = p.FH * p.FW;
            const bool has_tiles = static_cast<int>(blockIdx.x) < p.total_tiles;
            float* obase = p.out + (static_cast<size_t>(blockIdx.x) * nsub + sub) * p.part_stride;
            for (int fw = 0; fw < FW; ++fw) {
                if (fw_base + fw >= p.FW) break;   // spare accumulator of the row's last tap group
                const int tap = fh * p.FW + fw_base + fw;
                for (int c = 0; c < p.NT; c += 32) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + fw * acc_cols + c;
                    tmem_ld_32x32(taddr, v);
                    tmem_ld_wait();
                    if (diag) {
                        if (sub) { tmem_ld_32x32(taddr + p.NT, v); tmem_ld_wait(); }   // second half tile: lower right quadrant
                    } else if (stacked) {
                        uint32_t w[32];
                        tmem_ld_32x32(taddr + p.NT, w);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 32; ++q) v[q] = __float_as_uint(__uint_as_float(v[q]) + __uint_as_float(w[q]));
                    }
                    if (oc < p.OC) {
                        float* dst = obase + (static_cast<size_t>(oc) * taps + tap) * p.IC + ic0 + c;
#pragma unroll
                        for (int q = 0; q < 32; q += 4) {
                            float4 o = has_tiles ? make_float4(__uint_as_float(v[q]), __uint_as_float(v[q + 1]),
                                                               __uint_as_float(v[q + 2]), __uint_as_float(v[q + 3]))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                            *reinterpret_cast<float4*>(dst + q) = o;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (prof_on && threadIdx.x == 0) {
        p.prof[kProfTotal] = static_cast<unsigned long long>(clock64() - t_kernel);
        p.prof[kProfTotal + 1] = globaltimer_ns() - ns_kernel;   // wall time of the same span, ns
    }
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

}  // namespace alpha
