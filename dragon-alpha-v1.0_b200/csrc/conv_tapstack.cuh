// Stride-1 forward conv / deltaX for few output channels in plain TF32: the taps of one filter row
// share ONE tcgen05.mma.
//
// An MMA of N columns keeps the tensor pipe busy for max(N / 2, ~59) clocks and reads its 128 x 8
// A operand (4 KB) from shared memory whatever N is, so with 64 output channels a tap-by-tap kernel
// pays 59 clocks and 6 KB of operand reads for 32 clocks of tensor work.  Here the W tiles of the FW
// taps of a filter row lie back to back in shared memory and form one B operand of FW * BN columns:
//
//     D[q][fw * BN + oc] += sum_ic  patch[q + fh * 32][ic] * W[oc][fh][fw][ic]
//
// where q runs over the 128 positions of a tile = 4 output rows x 32 patch columns.  The A operand
// is not shifted by fw; instead every output pixel gathers its FW partial sums from FW neighbouring
// accumulator lanes:  Y[r][c] = sum_fw D[r * 32 + c + fw][fw * BN + oc].  A tile row holds CB <=
// 32 - (FW - 1) output columns plus the FW - 1 halo columns, so the neighbours are lanes of the same
// warp and the gather is FW - 1 warp shuffles per value.
//
// All of W (kchunks x FH x FW tiles of BN x 32 floats) stays resident in shared memory; only the
// input patches (32 channels x 32 columns x (4 + FH - 1) rows, zero-filled outside the image by the
// TMA) stream through a ring.  Tensor memory holds two accumulators (2 x FW * BN columns), so the
// gather / store of one tile overlaps the MMAs of the next.
//
// Two issuing threads: in a kernel one thread gets a tcgen05.mma started only every 100-120 clocks
// (waits, fences and commits run in series with its MMAs), more than the 96 clocks an MMA of 192
// columns keeps the pipe busy.  Issuer i owns accumulator i and every second tile of the CTA, so
// each accumulator still sees one thread and one fixed order of MMAs (results are reproducible),
// and the patches of two tiles are in use at a time.
//
// The epilogue uses no shared memory: after the gather a lane holds 32 channels of ONE pixel; a
// 4 x 4 transpose of 16-byte pieces among groups of four lanes (two shuffle stages) leaves it with
// 16 bytes of FOUR pixels, so that a store instruction writes 64 contiguous bytes per pixel.
//
// Warps: 0 TMA producer, 1 and 10 MMA issuers (1 owns tensor memory), 2-9 epilogue (two warps per
// tensor-memory lane quadrant, each with half of the channels).
#pragma once
#include "conv_halo.cuh"

namespace alpha {

constexpr int kTapStackThreads = 352;   // warps: 0 TMA, 1 and 10 MMA, 2-9 epilogue

struct TapStackParams {
    float* out;          // [N][OH][OW][ldo]
    const float* bias;   // [Ncols] or nullptr
    int act_on;          // 1: LeakyReLU with slope act_k after the bias
    float act_k;
    int* status;
    unsigned long long* prof;  // optional cycle counters of CTA 0 (nullptr = off), slots of HaloProf
    int N, OH, OW;
    int Ncols, ldo;      // Ncols % 4 == 0
    int FH, FW, pad_h, pad_w;
    int kchunks;         // reduction channels / 32
    int BN;              // accumulator columns per tap: Ncols rounded up to 16
    int CB;              // output columns per tile row, <= 32 - (FW - 1)
    int row_blocks, col_blocks, total_tiles;
    int npb;             // patch ring slots
    uint32_t patch_bytes;   // (4 + FH - 1) * 4096
    uint32_t w_tile;        // BN * 128: one tap of one 32-channel chunk
    uint32_t w_bytes;       // kchunks * FH * FW * w_tile
    uint32_t accw;          // FW * BN columns per accumulator
    uint32_t idesc, tmem_cols;
};

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets row (lane base + t).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// 32 channels of one tile row: Y[c] = sum over fw of D[lane + fw][fw * BN + channel], the partial sums of the
// FW taps gathered from the next lanes.  FW_T = 2 or 3 issues all loads before one wait; FW_T = 0 is any FW.
template <int FW_T>
__device__ __forceinline__ void tapstack_gather(uint32_t tcol, int BN, int FW, uint32_t (&y)[32])
{
    const unsigned full = 0xffffffffu;
    if constexpr (FW_T == 3) {
        uint32_t b[32], c[32];
        tmem_ld_32x32(tcol, y);
        tmem_ld_32x32(tcol + BN, b);
        tmem_ld_32x32(tcol + 2 * BN, c);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 32; ++q)
            y[q] = __float_as_uint((__uint_as_float(y[q]) + __shfl_down_sync(full, __uint_as_float(b[q]), 1)) +
                                   __shfl_down_sync(full, __uint_as_float(c[q]), 2));
    } else if constexpr (FW_T == 2) {
        uint32_t b[32];
        tmem_ld_32x32(tcol, y);
        tmem_ld_32x32(tcol + BN, b);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 32; ++q)
            y[q] = __float_as_uint(__uint_as_float(y[q]) + __shfl_down_sync(full, __uint_as_float(b[q]), 1));
    } else {
        tmem_ld_32x32(tcol, y);
        tmem_ld_wait();
        for (int fw = 1; fw < FW; ++fw) {
            uint32_t v[32];
            tmem_ld_32x32(tcol + fw * BN, v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 32; ++q)
                y[q] = __float_as_uint(__uint_as_float(y[q]) + __shfl_down_sync(full, __uint_as_float(v[q]), fw));
        }
    }
}

// 4 x 4 transpose of 16-byte pieces among the four lanes 4k .. 4k + 3: on entry a[j] is piece j of this lane's
// pixel, on return a[j] is piece (lane & 3) of the pixel of lane 4k + j.
__device__ __forceinline__ void transpose4_lanes(float4 (&a)[4], int lane)
{
    const unsigned full = 0xffffffffu;
    const bool b0 = lane & 1, b1 = lane & 2;
#pragma unroll
    for (int m = 0; m < 4; m += 2) {
        // lanes with bit 0 clear give away their odd piece and receive the partner's even one, and vice versa
        float4 s = b0 ? a[m] : a[m + 1];
        s.x = __shfl_xor_sync(full, s.x, 1); s.y = __shfl_xor_sync(full, s.y, 1);
        s.z = __shfl_xor_sync(full, s.z, 1); s.w = __shfl_xor_sync(full, s.w, 1);
        if (b0) a[m] = s; else a[m + 1] = s;
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float4 s = b1 ? a[m] : a[m + 2];
        s.x = __shfl_xor_sync(full, s.x, 2); s.y = __shfl_xor_sync(full, s.y, 2);
        s.z = __shfl_xor_sync(full, s.z, 2); s.w = __shfl_xor_sync(full, s.w, 2);
        if (b1) a[m] = s; else a[m + 2] = s;
    }
}

template <int FW_T, int FH_T>
__global__ void __launch_bounds__(kTapStackThreads, 1)
    conv_tapstack_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const TapStackParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* wres = smem;                                                   // resident W tiles
    uint8_t* patches = wres + p.w_bytes;                                    // ring of input patches
    uint64_t* bars = reinterpret_cast<uint64_t*>(patches + static_cast<size_t>(p.npb) * p.patch_bytes);
    uint64_t* w_full = bars;
    uint64_t* patch_full = w_full + 1;
    uint64_t* patch_empty = patch_full + p.npb;
    uint64_t* acc_full = patch_empty + p.npb;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int i = 0; i < p.npb; ++i) {
            mbar_init(&patch_full[i], 1);
            mbar_init(&patch_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 256);
        }
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int per_img = p.row_blocks * p.col_blocks;
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0;
    const long long t_kernel = clock64();
    const uint32_t w_a = smem_u32(wres), patches_a = smem_u32(patches);
    const uint32_t wfull_a = smem_u32(w_full), pfull_a = smem_u32(patch_full), pempty_a = smem_u32(patch_empty);
    const uint32_t afull_a = smem_u32(acc_full), aempty_a = smem_u32(acc_empty);

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: all of W once, then the patches of this CTA's tiles ----
            mbar_arrive_expect_tx_a(wfull_a, p.w_bytes);
            for (int c = 0; c < p.kchunks; ++c)
                for (int tap = 0; tap < p.FH * p.FW; ++tap)
                    tma_load_3d_a(w_a + (c * p.FH * p.FW + tap) * p.w_tile, &tmB, wfull_a, c * 32, tap, 0);
            RingPos pp;
            bool ok = true;
            unsigned long long w_patch = 0;
            for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                const int n = t / per_img;
                const int r = t - n * per_img;
                const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
                const int h0 = rb * 4 - p.pad_h, w0 = cb * p.CB - p.pad_w;
                for (int c = 0; c < p.kchunks; ++c) {
                    if (!wait_prof(pempty_a + 8 * pp.idx, pp.phase ^ 1, prof_on, w_patch)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                    mbar_arrive_expect_tx_a(pfull_a + 8 * pp.idx, p.patch_bytes);
                    tma_load_4d_a(patches_a + pp.idx * p.patch_bytes, &tmA, pfull_a + 8 * pp.idx, c * 32, w0, h0, n);
                    pp.advance(p.npb);
                }
            }
            if (prof_on) p.prof[kProfProducerPatchWait] = w_patch;
        }
        __syncwarp();
    } else if (warp == 1 || warp == 10) {
        if (lane == 0) {
            // ---- MMA issuers: issuer `which` owns accumulator `which` and the tiles j = which, which + 2, ... of
            // this CTA (tile j = blockIdx.x + j * gridDim.x); chunk c of tile j is load number j * kchunks + c ----
            const uint32_t which = warp == 1 ? 0u : 1u;
            const bool prof_me = prof_on && which == 0;
            RingPos pp;
            for (uint32_t i = 0; i < which * p.kchunks; ++i) pp.advance(p.npb);
            uint32_t acc_phase = 0;
            unsigned long long w_patch = 0, w_b = 0, w_acc = 0;
            const long long t_begin = clock64();
            bool ok = wait_prof(wfull_a, 0, prof_me, w_b);
            if (!ok) report(p.status, kStatusMmaTimeout);
            tc_fence_after_sync();
            const uint32_t dhi = smem_desc_hi(1024, kSwizzle128B);   // both operands: K-major rows of 128 B, 8-row groups 1024 B apart
            const uint32_t w_lo0 = smem_desc_lo(w_a, 16), patch_lo0 = smem_desc_lo(patches_a, 16);
            const uint32_t w_row16 = (p.FW * p.w_tile) >> 4;         // the FW tiles of one filter row
            const uint32_t patch16 = p.patch_bytes >> 4;
            const uint32_t idesc = p.idesc;
            const uint32_t d = tmem_base + which * p.accw;
            const uint32_t my_full = afull_a + 8 * which, my_empty = aempty_a + 8 * which;
            for (long long t = blockIdx.x + static_cast<long long>(which) * gridDim.x; t < p.total_tiles && ok; t += 2ll * gridDim.x) {
                if (!wait_prof(my_empty, acc_phase ^ 1, prof_me, w_acc)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                tc_fence_after_sync();
                uint32_t acc = 0u;
                uint32_t b_row = w_lo0;
                for (int c = 0; c < p.kchunks && ok; ++c) {
                    if (!wait_prof(pfull_a + 8 * pp.idx, pp.phase, prof_me, w_patch)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after_sync();
                    uint32_t a_row = patch_lo0 + pp.idx * patch16;
                    // one patch row = 32 positions = 4096 B = 256 descriptor units
                    if constexpr (FH_T > 0) {
                        // straight-line issue: a branch between two MMAs costs the issuing thread tens of clocks
                        static_for<0, FH_T>([&](auto fh_) {
                            constexpr uint32_t fh = decltype(fh_)::value;
                            const uint32_t b_fh = b_row + fh * w_row16;
                            static_for<0, 4>([&](auto kk_) {
                                constexpr uint32_t kk = decltype(kk_)::value;
                                mma_tf32_ss2_imm<fh * 256u + kk * 2u, kk * 2u>(d, a_row, dhi, b_fh, dhi, idesc, (fh == 0 && kk == 0) ? acc : 1u);
                            });
                        });
                        acc = 1u;
                        b_row += FH_T * w_row16;
                    } else {
                        for (int fh = 0; fh < p.FH; ++fh, a_row += 256u, b_row += w_row16) {
#pragma unroll
                            for (uint32_t kk = 0; kk < 4; ++kk) {
                                mma_tf32_ss2(d, a_row + kk * 2u, dhi, b_row + kk * 2u, dhi, idesc, acc);
                                acc = 1u;
                            }
                        }
                    }
                    mma_commit_a(pempty_a + 8 * pp.idx);
                    pp.advance(p.npb);
                }
                mma_commit_a(my_full);
                acc_phase ^= 1u;
                for (int i = 0; i < p.kchunks; ++i) pp.advance(p.npb);   // the other issuer's tile
            }
            if (prof_me) {
                p.prof[kProfMmaPatchWait] = w_patch; p.prof[kProfMmaBWait] = w_b; p.prof[kProfMmaAccWait] = w_acc;
                p.prof[kProfMmaTotal] = static_cast<unsigned long long>(clock64() - t_begin);
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..9.  Warp w reads tensor-memory lanes 32 * (w % 4) ... = one tile row; warps
        // 2..5 take the channels [0, 32), [64, 96), ... of that row, warps 6..9 the channels [32, 64), ... ----
        const int quad = warp & 3, half = (warp - 2) >> 2;
        RingPos ap;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        unsigned long long w_acc = 0;
        const long long t_begin = clock64();
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
            if (!wait_prof(afull_a + 8 * ap.idx, ap.phase, prof_on, w_acc)) { report(p.status, kStatusEpilogueTimeout); break; }
            tc_fence_after_sync();
            const int n = t / per_img;
            const int r = t - n * per_img;
            const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
            const int oh = rb * 4 + quad, ow0 = cb * p.CB;
            const bool row_ok = oh < p.OH;
            float* orow = p.out + (static_cast<size_t>(n) * p.OH + (row_ok ? oh : 0)) * p.OW * p.ldo + static_cast<size_t>(ow0) * p.ldo;
            const uint32_t tcol = lane_base + ap.idx * p.accw;
            bool released = false;
            for (int c0 = half * 32; c0 < p.Ncols; c0 += 64) {
                uint32_t y[32];
                tapstack_gather<FW_T>(tcol + c0, p.BN, p.FW, y);
                if (c0 + 64 >= p.Ncols) {
                    // everything this warp needs of the accumulator is in registers: hand it back to the MMA warp
                    tc_fence_before_sync();
                    mbar_arrive_a(aempty_a + 8 * ap.idx);
                    released = true;
                }
                // bias and activation on this lane's pixel, then the lane transpose and the stores: slot j of lane
                // 4k + i ends up with channels [4i, 4i + 4) of a 16-channel group of the pixel of lane 4k + j
                const int li = lane & 3, px0 = lane & ~3;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int ch = c0 + h * 16;
                    float4 a[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        a[q] = make_float4(__uint_as_float(y[h * 16 + 4 * q]), __uint_as_float(y[h * 16 + 4 * q + 1]),
                                           __uint_as_float(y[h * 16 + 4 * q + 2]), __uint_as_float(y[h * 16 + 4 * q + 3]));
                        if (p.bias && ch + 4 * q < p.Ncols) {
                            const float4 b = *reinterpret_cast<const float4*>(p.bias + ch + 4 * q);
                            a[q].x += b.x; a[q].y += b.y; a[q].z += b.z; a[q].w += b.w;
                        }
                        if (p.act_on) leaky_relu4(a[q], p.act_k);
                    }
                    transpose4_lanes(a, lane);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int px = px0 + j;
                        if (row_ok && px < p.CB && ow0 + px < p.OW && ch + 4 * li < p.Ncols)
                            *reinterpret_cast<float4*>(orow + static_cast<size_t>(px) * p.ldo + ch + 4 * li) = a[j];
                    }
                }
            }
            if (!released) {
                tc_fence_before_sync();
                mbar_arrive_a(aempty_a + 8 * ap.idx);
            }
            ap.advance(2);
        }
        if (prof_on && threadIdx.x == 64) {
            p.prof[kProfEpiWait] = w_acc;
            p.prof[kProfEpiWork] = static_cast<unsigned long long>(clock64() - t_begin) - w_acc;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (prof_on && threadIdx.x == 0) p.prof[kProfTotal] = static_cast<unsigned long long>(clock64() - t_kernel);
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

}  // namespace alpha
