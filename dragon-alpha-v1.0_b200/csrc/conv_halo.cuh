// Stride-1 forward conv / deltaX with each input tile fetched once.
//
// A persistent CTA walks macro tiles of JH x JW accumulators; one accumulator is 16 output rows x 8
// output columns (128 tensor-memory lanes).  For every 32-channel chunk the CTA loads the input
// patch that the macro tile needs - (16*JH + FH - 1) rows x (8*JW + FW - 1) columns of pixels,
// 128 bytes each, zero-filled outside the image by the TMA - exactly once, and forms the A operand
// of every filter tap as a shared-memory descriptor that starts (fh*PW + fw) pixel rows into the
// patch: tcgen05 applies the 128-byte swizzle to absolute shared-memory addresses, so a descriptor
// may start at any 128-byte row of a TMA-written tile, and the stride between groups of 8 rows
// (SBO) is simply the patch pitch.  B tiles (one filter tap x 32 channels x BN) stream through a
// ring.  In 3xTF32 mode four warps rewrite each landed patch as hi/lo planes once; the weights
// arrive pre-split.  3xTF32 has two forms: mode3x == 1 issues lo*hi, hi*lo and hi*hi as three MMAs
// of BN columns into one accumulator; mode3x == 2 ("wide", for BN <= 64, where an MMA of 64 columns
// costs almost as much as one of 128) issues hi x [hi | lo] as ONE MMA of 2*BN columns - the lo
// plane of a B tile directly follows its hi plane in shared memory - plus lo x hi into the second
// half of those columns, and the epilogue adds the two column halves of the accumulator.
// Accumulators are double-buffered in tensor memory when they fit, so the epilogue of one macro
// tile overlaps the loads and MMAs of the next.
//
// Warps: 0 TMA producer, 1 and 10 MMA issuers (1 owns tensor memory), 2-5 epilogue, 6-9 operand split.
//
// Two issuers (p.dual): one thread can start a tcgen05.mma only every ~59 clocks and pays the
// barrier wait, fence and commit of every stage in series with its MMAs.  The W-tile stages of the
// ring alternate between two issuing threads that accumulate into the same tensor-memory columns
// (stage s belongs to issuer s & 1; the ring has an even number of slots, so every slot and its
// barriers always meet the same issuer, in order).  The issuer of a tile's first stage overwrites
// the accumulator and then releases a "tile started" barrier that the other one waits for before
// its first MMA of the tile; patch-empty and accumulator-full collect the commits of both.
// The host turns this on for plain TF32 only (N = 64..128 per MMA, where the issue interval and
// not the tensor pipe is the bound).  The order in which the two issuers' MMAs reach the pipe
// depends on timing, so the fp32 accumulation order, and with it the last bits of a TF32 result,
// can differ between runs; the 3xTF32 forms keep one issuer and a fixed order.
//
// One tcgen05.mma of this shape takes 59-128 clocks of its issuing thread, so the issue
// loop is kept free of divisions, pointer conversions and per-iteration address arithmetic: ring
// positions are counters, barriers and tiles are 32-bit shared-memory addresses, descriptors are a
// constant high half plus a low half that only gets small additions.
#pragma once
#include "conv_kernels.cuh"

namespace alpha {

constexpr int kHaloThreads = 320;    // CTA-pair kernel: warps 0 TMA, 1 MMA, 2-5 epilogue, 6-9 split
constexpr int kHaloThreads2 = 352;   // single-CTA kernel: one more warp (10) as second MMA issuer

// Slots of the optional cycle counters (clock64 ticks of CTA 0, summed over the launch).
enum HaloProf {
    kProfProducerPatchWait = 0, kProfProducerBWait, kProfMmaPatchWait, kProfMmaBWait, kProfMmaAccWait,
    kProfMmaTotal, kProfEpiWait, kProfEpiWork, kProfSplitWait, kProfSplitWork, kProfTotal, kProfSlots = 16
};

struct HaloParams {
    float* out;          // [N][OH][OW][ldo]
    const float* bias;   // [Ncols] or nullptr
    int act_on;          // 1: LeakyReLU with slope act_k after the bias
    float act_k;
    int* status;
    unsigned long long* prof;  // optional cycle counters of CTA 0 (nullptr = off), see HaloProf
    int N, OH, OW;       // output geometry
    int Ncols, ldo;
    int FH, FW, pad_h, pad_w;
    int kchunks;         // reduction channels / 32
    int BN, n_tiles;
    int JH, JW;          // accumulators per macro tile, vertically and horizontally
    int PH, PW;          // patch rows and columns (pixels)
    int row_blocks, col_blocks;
    int NI, SG;          // images stacked in one accumulator (small images) and rows per image slot
    int n_blocks;        // ceil(N / NI)
    int total_tiles;     // n_tiles * n_blocks * row_blocks * col_blocks
    int npb, sb;         // patch buffers, B ring stages
    int acc_bufs;        // 1 or 2 accumulator sets
    int mode3x, b_mn, flip;   // mode3x: 0 plain TF32, 1 three MMAs, 2 wide B
    int dual;                 // 1: two MMA-issuing threads take alternate W-tile stages (sb is even)
    int split_b;              // 3xTF32: 1 = only the hi plane of every W tile is loaded and the split warps form its lo
                              // plane in shared memory (1x1 products, whose W traffic from L2 is what binds them)
    int flat, flat_rb4, flat_total;   // flat = 1: accumulators of 4 output rows x 32 patch columns, each with its own patch of
                              // FH + 3 rows x 32 pixels (images at most 30 pixels wide); macro tile t holds the accumulators
                              // t * J ... of the flat_total = N * flat_rb4 four-row blocks of the batch (flat_rb4 per image)
    int w_img_rows;           // > 0: every image has its own W (batched matrix products); rows of W per image, added to the
                              // row coordinate of every W tile (stacked images and split-K are then off)
    int ksplit, cps;          // split-K: every tile is computed as ksplit partial sums over cps reduction chunks each;
                              // partial sp of image n is stored as image sp * N + n of the output map
    uint32_t idesc, idesc_wide, tmem_cols;   // idesc_wide: N = 2 * BN
    uint32_t patch_bytes;  // one plane of one patch buffer, multiple of 1024
    uint32_t patch_tx;     // bytes one patch load delivers
    uint32_t b_bytes;      // one plane of one B stage, multiple of 1024
    uint32_t b_tx;
};

// Bounded wait that also charges the waited cycles to a counter when profiling is on.
__device__ __forceinline__ bool wait_prof(uint32_t bar, uint32_t parity, bool prof, unsigned long long& acc)
{
    if (!prof) return mbar_wait_a(bar, parity);
    // try_wait itself may suspend the thread for a while, so the whole call is timed
    const long long t0 = clock64();
    const bool ok = mbar_wait_a(bar, parity);
    acc += static_cast<unsigned long long>(clock64() - t0);
    return ok;
}

// Virtual tile v -> tile t and the range of reduction chunks [c0, c1) of its split-K part sp.
struct TilePart { int t, sp, c0, c1; };
__device__ __forceinline__ TilePart tile_part(const HaloParams& p, int v)
{
    TilePart r{v, 0, 0, p.kchunks};
    if (p.ksplit > 1) {
        r.t = v / p.ksplit;
        r.sp = v - r.t * p.ksplit;
        r.c0 = r.sp * p.cps;
        r.c1 = r.c0 + p.cps < p.kchunks ? r.c0 + p.cps : p.kchunks;
    }
    return r;
}

// The four K=8 steps of one 32-channel chunk into one accumulator.  MODE 0: 4 MMAs; 1: 12 MMAs
// (three per step); 2: 8 MMAs (hi x [hi | lo] over 2*BN columns, then lo x hi over BN columns).
template <int MODE>
__device__ __forceinline__ void issue_chunk(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t b_kstep, uint32_t a_lo_off, uint32_t b_lo_off, uint32_t idesc,
                                            uint32_t idesc_wide, uint32_t acc_first, uint32_t side_off = 0)
{
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const uint32_t a_k = a_lo + kk * 2, b_k = b_lo + kk * b_kstep;
        const uint32_t acc = kk == 0 ? acc_first : 1u;
        if (MODE == 1) {
            mma_tf32_ss2(d, a_k + a_lo_off, a_hi, b_k, b_hi, idesc, acc);
            mma_tf32_ss2(d, a_k, a_hi, b_k + b_lo_off, b_hi, idesc, 1u);
            mma_tf32_ss2(d, a_k, a_hi, b_k, b_hi, idesc, 1u);
        } else if (MODE == 2) {
            // hi*hi lands in columns [0, BN); both correction terms go to the side columns [BN, 2*BN):
            // tensor-core accumulation truncates, so every MMA into the main sum costs up to one ulp
            // of it, while truncation in the side sum is 2^-11 times smaller
            mma_tf32_ss2(d, a_k, a_hi, b_k, b_hi, idesc_wide, acc);
            mma_tf32_ss2(d + side_off, a_k + a_lo_off, a_hi, b_k, b_hi, idesc, 1u);
        } else {
            mma_tf32_ss2(d, a_k, a_hi, b_k, b_hi, idesc, acc);
        }
    }
}

// Descriptor constants of the issue loop.
struct IssueConsts {
    uint32_t a_dhi, b_dhi, b_kstep, a_lo_off, b_lo_off, idesc, idesc_wide, accw;
};

// Static specialisations (K-major W tiles only): every descriptor offset is a compile-time constant
// handed to the MMA wrapper as an immediate, so a stage costs the issuing thread a handful of
// additions up front and nothing between MMAs.
//
// The four K=8 steps of one 32-channel chunk into one accumulator; A_OFF = offset of the tap and
// accumulator inside the patch (16-byte units).  a / a_lo: hi and lo plane of the patch row,
// b / b_lo: hi and lo plane of the tap's W tile, d / d_side: main and side accumulator columns.
template <int MODE, uint32_t A_OFF>
__device__ __forceinline__ void issue_chunk_imm(uint32_t d, uint32_t d_side, uint32_t a, uint32_t a_lo, uint32_t a_hi, uint32_t b,
                                                uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t idesc_wide,
                                                uint32_t acc_first)
{
    static_for<0, 4>([&](auto kk_) {
        constexpr uint32_t kk = decltype(kk_)::value;
        const uint32_t acc = kk == 0 ? acc_first : 1u;
        if constexpr (MODE == 1) {
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d, a_lo, a_hi, b, b_hi, idesc, acc);
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d, a, a_hi, b_lo, b_hi, idesc, 1u);
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d, a, a_hi, b, b_hi, idesc, 1u);
        } else if constexpr (MODE == 2) {
            // hi*hi lands in columns [0, BN); both correction terms go to the side columns [BN, 2*BN):
            // tensor-core accumulation truncates, so every MMA into the main sum costs up to one ulp
            // of it, while truncation in the side sum is 2^-11 times smaller
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d, a, a_hi, b, b_hi, idesc_wide, acc);
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d_side, a_lo, a_hi, b, b_hi, idesc, 1u);
        } else {
            mma_tf32_ss2_imm<A_OFF + kk * 2, kk * 2>(d, a, a_hi, b, b_hi, idesc, acc);
        }
    });
}

// One filter tap into the JH_T x JW_T accumulators of a macro tile.  a_row / a_row_lo: descriptor
// low halves of the patch row of this filter row (hi / lo plane); TAP_OFF = fw * 8.
// FLAT_T: accumulator j reads its own patch, 6 rows x 32 pixels x 128 B = 1536 descriptor units after the previous one.
template <int MODE, int JH_T, int JW_T, uint32_t kPW8, uint32_t TAP_OFF, bool FLAT_T = false>
__device__ __forceinline__ void issue_tap(uint32_t d0, uint32_t a_row, uint32_t a_row_lo, uint32_t bl, const IssueConsts& k,
                                          uint32_t acc_first)
{
    const uint32_t bl_lo = bl + k.b_lo_off;
    static_for<0, JH_T * JW_T>([&](auto j_) {
        constexpr uint32_t j = decltype(j_)::value, jh = j / JW_T, jw = j % JW_T;
        constexpr uint32_t a_off = FLAT_T ? TAP_OFF + j * 1536u : TAP_OFF + jh * 16 * kPW8 + jw * 64;
        const uint32_t d = d0 + j * k.accw;
        issue_chunk_imm<MODE, a_off>(d, d + (k.accw >> 1), a_row, a_row_lo, k.a_dhi, bl, bl_lo, k.b_dhi,
                                     k.idesc, k.idesc_wide, acc_first);
    });
}

// The FW_T taps of one filter row (B stage holds them back to back, b_tile16 apart).
template <int MODE, int FW_T, int JH_T, int JW_T, uint32_t kPW8, bool FLAT_T = false>
__device__ __forceinline__ void issue_row(uint32_t d0, uint32_t a_row, uint32_t bl, uint32_t b_tile16, const IssueConsts& k,
                                          uint32_t acc_first)
{
    const uint32_t a_row_lo = a_row + k.a_lo_off;
    static_for<0, FW_T>([&](auto fw_) {
        constexpr uint32_t fw = decltype(fw_)::value;
        issue_tap<MODE, JH_T, JW_T, kPW8, fw * 8, FLAT_T>(d0, a_row, a_row_lo, bl + fw * b_tile16, k, fw == 0 ? acc_first : 1u);
    });
}

// FW_T > 0 selects a specialisation with compile-time FW, JH and JW whose MMAs are issued as
// straight-line code with immediate descriptor offsets; with ROW_T one B stage holds the FW taps of
// one filter row, otherwise one tap.  FW_T == 0 is the generic form: any filter, one tap per stage.
// FLAT_T (static forms only): the JH_T * JW_T accumulators are flat tiles of 4 rows x 32 patch columns, see HaloParams::flat.
template <int FW_T, int JH_T, int JW_T, bool ROW_T, bool FLAT_T = false>
__global__ void __launch_bounds__(kHaloThreads2, 1)
    conv_halo_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmO,
                     const HaloParams p)
{
    constexpr bool kStatic = FW_T > 0;
    constexpr bool kRow = kStatic && ROW_T;
    const int tps = kRow ? FW_T : 1;              // taps per B stage
    const int stages_per_chunk = kRow ? p.FH : p.FH * p.FW;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t planes = p.mode3x ? 2u : 1u;
    const uint32_t patch_stride = p.patch_bytes * planes;
    const uint32_t b_tile = p.b_bytes * planes;   // hi (+ lo) planes of one tap
    const uint32_t b_stride = b_tile * tps;       // one ring stage
    uint8_t* patches = smem;
    uint8_t* bring = smem + static_cast<size_t>(p.npb) * patch_stride;
    uint8_t* staging = bring + static_cast<size_t>(p.sb) * b_stride;   // 2 x 16 KB epilogue slabs
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * 16384);
    uint64_t* patch_full = bars;
    uint64_t* patch_ready = patch_full + p.npb;
    uint64_t* patch_empty = patch_ready + p.npb;
    uint64_t* b_full = patch_empty + p.npb;
    uint64_t* b_ready = b_full + p.sb;
    uint64_t* b_empty = b_ready + p.sb;
    uint64_t* acc_full = b_empty + p.sb;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* tile_started = acc_empty + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tile_started + 2);

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.npb; ++i) {
            mbar_init(&patch_full[i], 1);
            mbar_init(&patch_ready[i], 128);
            mbar_init(&patch_empty[i], p.dual ? 2 : 1);
        }
        for (int i = 0; i < p.sb; ++i) {
            mbar_init(&b_full[i], 1);
            mbar_init(&b_ready[i], 128);
            mbar_init(&b_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], p.dual ? 2 : 1);
            mbar_init(&acc_empty[i], 128);
            mbar_init(&tile_started[i], 1);
        }
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        prefetch_tmap(&tmBlo);
        prefetch_tmap(&tmO);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int J = p.JH * p.JW;
    const int per_img = p.row_blocks * p.col_blocks;
    const int vtiles = p.total_tiles * (p.ksplit > 1 ? p.ksplit : 1);
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0;
    const long long t_kernel = clock64();

    // 32-bit shared-memory addresses of everything the loops touch
    const uint32_t patches_a = smem_u32(patches), bring_a = smem_u32(bring);
    const uint32_t pfull_a = smem_u32(patch_full), pready_a = smem_u32(patch_ready), pempty_a = smem_u32(patch_empty);
    const uint32_t bfull_a = smem_u32(b_full), bempty_a = smem_u32(b_empty);
    const uint32_t afull_a = smem_u32(acc_full), aempty_a = smem_u32(acc_empty);

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            RingPos pp, bp;
            bool ok = true;
            unsigned long long w_patch = 0, w_b = 0;
            const int taps = p.FH * p.FW;
            for (int v = blockIdx.x; v < vtiles && ok; v += gridDim.x) {
                const TilePart tp = tile_part(p, v);
                const int t = tp.t;
                const int tn = t / (p.n_blocks * per_img);
                int r = t - tn * (p.n_blocks * per_img);
                const int nb = r / per_img;
                r -= nb * per_img;
                const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
                const int h0 = rb * 16 * p.JH - p.pad_h, w0 = cb * 8 * p.JW - p.pad_w;
                const int n = nb * p.NI;
                const int oc0 = tn * p.BN;
                const int wrow0 = n * p.w_img_rows;   // first W row of this image's own weights (0: shared weights)
                for (int c = tp.c0; c < tp.c1 && ok; ++c) {
                    if (!wait_prof(pempty_a + 8 * pp.idx, pp.phase ^ 1, prof_on, w_patch)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                    mbar_arrive_expect_tx_a(pfull_a + 8 * pp.idx, p.patch_tx);
                    if (FLAT_T) {
                        // one patch per accumulator; rb is the macro tile's index, a block past the end repeats the last one
                        const uint32_t sub = p.patch_tx / static_cast<uint32_t>(J);
                        for (int j = 0; j < J; ++j) {
                            int a = rb * J + j;
                            if (a >= p.flat_total) a = p.flat_total - 1;
                            const int an = a / p.flat_rb4, arb = a - an * p.flat_rb4;
                            tma_load_4d_a(patches_a + pp.idx * patch_stride + j * sub, &tmA, pfull_a + 8 * pp.idx, c * 32, -p.pad_w,
                                          arb * 4 - p.pad_h, an);
                        }
                    } else {
                        tma_load_4d_a(patches_a + pp.idx * patch_stride, &tmA, pfull_a + 8 * pp.idx, c * 32, w0, h0, n);
                    }
                    pp.advance(p.npb);
                    for (int st = 0; st < stages_per_chunk; ++st) {
                        if (!wait_prof(bempty_a + 8 * bp.idx, bp.phase ^ 1, prof_on, w_b)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                        const uint32_t bar = bfull_a + 8 * bp.idx;
                        mbar_arrive_expect_tx_a(bar, p.b_tx * tps * (p.split_b ? 1u : planes));
                        for (int q = 0; q < tps; ++q) {
                            const int tap = st * tps + q;
                            const uint32_t b_dst = bring_a + bp.idx * b_stride + q * b_tile;
                            if (!p.b_mn) {
                                tma_load_3d_a(b_dst, &tmB, bar, c * 32, tap, oc0 + wrow0);
                                if (p.mode3x && !p.split_b) tma_load_3d_a(b_dst + p.b_bytes, &tmBlo, bar, c * 32, tap, oc0 + wrow0);
                            } else {
                                const int tapw = p.flip ? (taps - 1 - tap) : tap;
                                for (int j = 0; j < p.BN / 32; ++j) {
                                    tma_load_3d_a(b_dst + j * 4096, &tmB, bar, oc0 + j * 32, tapw, c * 32 + wrow0);
                                    if (p.mode3x) tma_load_3d_a(b_dst + p.b_bytes + j * 4096, &tmBlo, bar, oc0 + j * 32, tapw, c * 32 + wrow0);
                                }
                            }
                        }
                        bp.advance(p.sb);
                    }
                }
            }
            if (prof_on) { p.prof[kProfProducerPatchWait] = w_patch; p.prof[kProfProducerBWait] = w_b; }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 10) {
        if (lane == 0 && (warp == 1 || p.dual)) {
            // ---- MMA issuer(s) ----
            const uint32_t which = warp == 1 ? 0u : 1u;
            const bool dual = p.dual != 0;
            const bool prof_on = p.prof != nullptr && blockIdx.x == 0 && which == 0;
            const uint32_t started_a = smem_u32(tile_started);
            uint32_t sg = 0;   // W-tile stages of this CTA so far; with two issuers stage sg belongs to issuer sg & 1
            RingPos pp, bp, ap;
            bool ok = true;
            unsigned long long w_patch = 0, w_b = 0, w_acc = 0;
            const long long t_begin = clock64();
            // descriptor halves that never change, and the steps of the low half (16-byte units)
            const uint32_t a_dhi = smem_desc_hi(FLAT_T ? 1024u : p.PW * 128, kSwizzle128B);
            const uint32_t b_dhi = p.b_mn ? smem_desc_hi(512, kSwizzle128B_Base32B) : smem_desc_hi(1024, kSwizzle128B);
            const uint32_t b_kstep = p.b_mn ? 64u : 2u;       // 1024 B or 32 B per K=8 step
            const uint32_t a_lo_off = p.patch_bytes >> 4;     // hi plane -> lo plane
            const uint32_t b_lo_off = p.b_bytes >> 4;
            const uint32_t row_step = p.PW * 8u;              // one patch row down
            const uint32_t jh_step = 16u * row_step;          // 16 patch rows down
            const uint32_t patch_lo0 = smem_desc_lo(patches_a, 16), patch_stride16 = patch_stride >> 4;
            const uint32_t bring_lo0 = smem_desc_lo(bring_a, p.b_mn ? 4096u : 16u), b_stride16 = b_stride >> 4;
            // weights arrive pre-split unless the split warps form the lo plane of the W tiles (split_b)
            const uint32_t pwait_a = p.mode3x ? pready_a : pfull_a, bwait_a = p.split_b ? smem_u32(b_ready) : bfull_a;
            const uint32_t accw = p.mode3x == 2 ? 2u * p.BN : p.BN;   // columns of one accumulator
            const uint32_t acc_cols = J * accw;
            const IssueConsts k{a_dhi, b_dhi, b_kstep, a_lo_off, b_lo_off, p.idesc, p.idesc_wide, accw};
            for (int v = blockIdx.x; v < vtiles && ok; v += gridDim.x) {
                const TilePart tp = tile_part(p, v);
                if (!wait_prof(aempty_a + 8 * ap.idx, ap.phase ^ 1, prof_on, w_acc)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d0 = tmem_base + ap.idx * acc_cols;
                // the issuer of the tile's first stage overwrites the accumulator; the other one must
                // not touch it before that MMA has been issued
                const bool owner = !dual || (sg & 1u) == which;
                uint32_t acc_first = owner ? 0u : 1u;
                bool announce = dual && owner, must_wait = dual && !owner;
                for (int c = tp.c0; c < tp.c1 && ok; ++c) {
                    if (!wait_prof(pwait_a + 8 * pp.idx, pp.phase, prof_on, w_patch)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                    tc_fence_after_sync();
                    uint32_t a_row = patch_lo0 + pp.idx * patch_stride16;
                    if constexpr (kRow) {
                        constexpr uint32_t kPW8 = FLAT_T ? 256u : (8 * JW_T + FW_T - 1) * 8;  // one patch row, in 16-byte units
                        const uint32_t b_tile16 = b_tile >> 4;
                        for (int fh = 0; fh < p.FH; ++fh, a_row += kPW8, bp.advance(p.sb)) {
                            if (dual && ((sg++) & 1u) != which) continue;   // the other issuer's stage
                            if (must_wait) {
                                if (!mbar_wait_a(started_a + 8 * ap.idx, ap.phase)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                                must_wait = false;
                                tc_fence_after_sync();
                            }
                            if (!wait_prof(bwait_a + 8 * bp.idx, bp.phase, prof_on, w_b)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                            tc_fence_after_sync();
                            const uint32_t bl = bring_lo0 + bp.idx * b_stride16;
                            if (p.mode3x == 1) issue_row<1, FW_T, JH_T, JW_T, kPW8, FLAT_T>(d0, a_row, bl, b_tile16, k, acc_first);
                            else if (p.mode3x == 2) issue_row<2, FW_T, JH_T, JW_T, kPW8, FLAT_T>(d0, a_row, bl, b_tile16, k, acc_first);
                            else issue_row<0, FW_T, JH_T, JW_T, kPW8, FLAT_T>(d0, a_row, bl, b_tile16, k, acc_first);
                            acc_first = 1u;
                            if (announce) { tc_fence_before_sync(); mbar_arrive_a(started_a + 8 * ap.idx); announce = false; }
                            mma_commit_a(bempty_a + 8 * bp.idx);
                        }
                    } else if constexpr (kStatic) {
                        constexpr uint32_t kPW8 = FLAT_T ? 256u : (8 * JW_T + FW_T - 1) * 8;
                        for (int fh = 0; fh < p.FH && ok; ++fh, a_row += kPW8) {
                            const uint32_t a_row_lo = a_row + a_lo_off;
                            static_for<0, FW_T>([&](auto fw_) {
                                constexpr uint32_t fw = decltype(fw_)::value;
                                if (!ok) return;
                                const bool take = !dual || ((sg++) & 1u) == which;
                                if (take) {
                                    if (must_wait) {
                                        if (!mbar_wait_a(started_a + 8 * ap.idx, ap.phase)) { report(p.status, kStatusMmaTimeout); ok = false; return; }
                                        must_wait = false;
                                        tc_fence_after_sync();
                                    }
                                    if (!wait_prof(bwait_a + 8 * bp.idx, bp.phase, prof_on, w_b)) { report(p.status, kStatusMmaTimeout); ok = false; return; }
                                    tc_fence_after_sync();
                                    const uint32_t bl = bring_lo0 + bp.idx * b_stride16;
                                    if (p.mode3x == 1) issue_tap<1, JH_T, JW_T, kPW8, fw * 8, FLAT_T>(d0, a_row, a_row_lo, bl, k, acc_first);
                                    else if (p.mode3x == 2) issue_tap<2, JH_T, JW_T, kPW8, fw * 8, FLAT_T>(d0, a_row, a_row_lo, bl, k, acc_first);
                                    else issue_tap<0, JH_T, JW_T, kPW8, fw * 8, FLAT_T>(d0, a_row, a_row_lo, bl, k, acc_first);
                                    acc_first = 1u;
                                    if (announce) { tc_fence_before_sync(); mbar_arrive_a(started_a + 8 * ap.idx); announce = false; }
                                    mma_commit_a(bempty_a + 8 * bp.idx);
                                }
                                bp.advance(p.sb);
                            });
                        }
                    } else {
                    for (int fh = 0; fh < p.FH && ok; ++fh, a_row += row_step) {
                        uint32_t a_tap = a_row;
                        for (int fw = 0; fw < p.FW; ++fw, a_tap += 8, bp.advance(p.sb)) {
                            if (dual && ((sg++) & 1u) != which) continue;   // the other issuer's stage
                            if (must_wait) {
                                if (!mbar_wait_a(started_a + 8 * ap.idx, ap.phase)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                                must_wait = false;
                                tc_fence_after_sync();
                            }
                            if (!wait_prof(bwait_a + 8 * bp.idx, bp.phase, prof_on, w_b)) { report(p.status, kStatusMmaTimeout); ok = false; break; }
                            tc_fence_after_sync();
                            const uint32_t bl = bring_lo0 + bp.idx * b_stride16;
                            uint32_t d = d0, a_jh = a_tap;
                            for (int jh = 0; jh < p.JH; ++jh, a_jh += jh_step) {
                                uint32_t a_j = a_jh;
                                for (int jw = 0; jw < p.JW; ++jw, a_j += 64, d += accw) {
                                    if (p.mode3x == 1) issue_chunk<1>(d, a_j, a_dhi, bl, b_dhi, b_kstep, a_lo_off, b_lo_off, p.idesc, p.idesc_wide, acc_first);
                                    else if (p.mode3x == 2) issue_chunk<2>(d, a_j, a_dhi, bl, b_dhi, b_kstep, a_lo_off, b_lo_off, p.idesc, p.idesc_wide, acc_first, accw >> 1);
                                    else issue_chunk<0>(d, a_j, a_dhi, bl, b_dhi, b_kstep, a_lo_off, b_lo_off, p.idesc, p.idesc_wide, acc_first);
                                }
                            }
                            acc_first = 1u;
                            if (announce) { tc_fence_before_sync(); mbar_arrive_a(started_a + 8 * ap.idx); announce = false; }
                            mma_commit_a(bempty_a + 8 * bp.idx);
                        }
                    }
                    }
                    mma_commit_a(pempty_a + 8 * pp.idx);
                    pp.advance(p.npb);
                }
                mma_commit_a(afull_a + 8 * ap.idx);
                ap.advance(p.acc_bufs);
            }
            if (prof_on) {
                p.prof[kProfMmaPatchWait] = w_patch; p.prof[kProfMmaBWait] = w_b; p.prof[kProfMmaAccWait] = w_acc;
                p.prof[kProfMmaTotal] = static_cast<unsigned long long>(clock64() - t_begin);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---- epilogue: warps 2..5, lane quadrant = warp % 4 ----
        const int quad = warp & 3;
        const int row = quad * 32 + lane;       // accumulator row = g*8 + i
        RingPos ap;
        unsigned long long w_acc = 0;
        const long long t_begin = clock64();
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const uint32_t stage_a = smem_u32(staging);
        uint32_t sbuf = 0;
        const bool wide = p.mode3x == 2;
        const uint32_t accw = wide ? 2u * p.BN : p.BN;
        for (int v = blockIdx.x; v < vtiles; v += gridDim.x) {
            const TilePart tp = tile_part(p, v);
            const int t = tp.t;
            if (!wait_prof(afull_a + 8 * ap.idx, ap.phase, prof_on, w_acc)) { report(p.status, kStatusEpilogueTimeout); break; }
            tc_fence_after_sync();
            const int tn = t / (p.n_blocks * per_img);
            int r = t - tn * (p.n_blocks * per_img);
            const int nb = r / per_img;
            r -= nb * per_img;
            const int rb = r / p.col_blocks, cb = r - rb * p.col_blocks;
            const int n = nb * p.NI;
            const int n0 = tn * p.BN;
            int j = 0;
            for (int jh = 0; jh < p.JH; ++jh)
                for (int jw = 0; jw < p.JW; ++jw, ++j) {
                    int oh0 = (rb * p.JH + jh) * 16, ow0 = (cb * p.JW + jw) * 8, n_img = n;
                    if (FLAT_T) {
                        const int a = rb * J + j;
                        if (a >= p.flat_total) continue;          // the repeated block of the last macro tile
                        n_img = a / p.flat_rb4;
                        oh0 = (a - n_img * p.flat_rb4) * 4;
                        ow0 = 0;
                    }
                    if (oh0 >= p.OH || ow0 >= p.OW) continue;  // accumulator entirely outside the image
                    const uint32_t tcol = lane_base + (ap.idx * J + j) * accw;
                    for (int c = 0; c < p.BN; c += 32) {
                        const int col0 = n0 + c;
                        if (col0 >= p.Ncols) break;
                        // slab `sbuf` was last read by the store issued two slabs ago
                        if (threadIdx.x == 64) tma_store_wait_read<1>();
                        named_barrier_sync(1, 128);
                        uint32_t v[32];
                        tmem_ld_32x32(tcol + c, v);
                        tmem_ld_wait();
                        if (wide) {
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
                            // 128-byte swizzle: 16-byte chunk q of row r lives at chunk q ^ (r & 7)
                            st_shared_v4(srow + ((q ^ (row & 7)) << 4), o);
                        }
                        fence_proxy_async_smem();
                        named_barrier_sync(1, 128);
                        if (threadIdx.x == 64) {
                            if (p.NI == 1) {
                                tma_store_4d_a(&tmO, stage_a + sbuf * 16384, col0, ow0, oh0, n_img + tp.sp * p.N);
                            } else {
                                // stacked images: image i starts SG groups (of 8 rows) further down the slab
                                for (int img = 0; img < p.NI; ++img)
                                    if (n + img < p.N)
                                        tma_store_4d_a(&tmO, stage_a + sbuf * 16384 + img * p.SG * 1024, col0, ow0, 0, n + img + tp.sp * p.N);
                            }
                            tma_store_commit();
                        }
                        sbuf ^= 1u;
                    }
                }
            tc_fence_before_sync();
            mbar_arrive_a(aempty_a + 8 * ap.idx);
            ap.advance(p.acc_bufs);
        }
        if (threadIdx.x == 64) tma_store_wait_all();  // the slabs must outlive their stores
        if (prof_on && threadIdx.x == 64) {
            p.prof[kProfEpiWait] = w_acc;
            p.prof[kProfEpiWork] = static_cast<unsigned long long>(clock64() - t_begin) - w_acc;
        }
    } else {
        // ---- operand split (3xTF32 only): warps 6..9 ----
        if (p.mode3x) {
            const int tid128 = threadIdx.x - 192;
            RingPos pp, bpos;
            bool ok = true;
            unsigned long long w_in = 0;
            const long long t_begin = clock64();
            for (int v = blockIdx.x; v < vtiles && ok; v += gridDim.x) {
                const TilePart tp = tile_part(p, v);
                for (int c = tp.c0; c < tp.c1 && ok; ++c) {
                    if (!wait_prof(pfull_a + 8 * pp.idx, pp.phase, prof_on, w_in)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                    uint8_t* ph = patches + static_cast<size_t>(pp.idx) * patch_stride;
                    split_plane_lo_x4(ph, ph + p.patch_bytes, p.patch_tx, tid128, 128);
                    fence_proxy_async_smem();
                    mbar_arrive_a(pready_a + 8 * pp.idx);
                    pp.advance(p.npb);
                    if (p.split_b) {
                        // the W-tile stages of this chunk, in the producer's order
                        for (int st = 0; st < stages_per_chunk && ok; ++st) {
                            if (!mbar_wait_a(bfull_a + 8 * bpos.idx, bpos.phase)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                            uint8_t* bt = bring + static_cast<size_t>(bpos.idx) * b_stride;
                            for (int q = 0; q < tps; ++q) split_plane_lo_x4(bt + q * b_tile, bt + q * b_tile + p.b_bytes, p.b_tx, tid128, 128);
                            fence_proxy_async_smem();
                            mbar_arrive_a(smem_u32(b_ready) + 8 * bpos.idx);
                            bpos.advance(p.sb);
                        }
                    }
                }
            }
            if (prof_on && threadIdx.x == 192) {
                p.prof[kProfSplitWait] = w_in;
                p.prof[kProfSplitWork] = static_cast<unsigned long long>(clock64() - t_begin) - w_in;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (prof_on && threadIdx.x == 0) p.prof[kProfTotal] = static_cast<unsigned long long>(clock64() - t_kernel);
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

}  // namespace alpha
