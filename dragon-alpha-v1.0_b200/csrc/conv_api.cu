// Host side of layer 1 of the C ABI: shape checks, tensor-map construction, tile choice, launches.
#include "../../include/alpha_conv_b200.h"
#include "conv_kernels.cuh"
#include "conv_halo.cuh"
#include "conv_halo_pair.cuh"
#include "conv_dw_halo.cuh"
#include "conv_tapstack.cuh"
#include "winograd.cuh"
#include "host_common.h"

#include <nvtx3/nvToolsExt.h>   // header-only: resolves a profiler's injection library at run time, no link dependency

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace alpha {

// ---- thread-local error text, process-wide settings ---------------------------------------------

static thread_local char g_err[512] = "";
static thread_local const char* g_last_algo = "";
static std::atomic<unsigned long long> g_launches{0};

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static thread_local char g_plan[128] = "";
// The calling thread is sizing a call (alpha_conv_workspace_bytes): scratch requests are added up
// and answered with a placeholder address; nothing is allocated, launched or copied.
static thread_local bool t_dry = false;

void note_launch(const char* algo)
{
    if (t_dry) return;
    g_last_algo = algo;
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

// ---- tuning options -----------------------------------------------------------------------------
//
// Every switch the planners consult lives in one table.  The environment (ALPHA_<NAME>) seeds the
// table once, at the first call into the library; afterwards alpha_conv_set_option() is the only
// way to change a value, so no call reads the environment on its way to a launch.
enum Opt {
    OPT_CONV_TILE,      // 0 = choose by cost model, 1 = always the per-tap im2col kernel, 2 = halo kernel wherever it applies
    OPT_CONV_DW,        // 1 = split-K im2col deltaW kernel even where the halo-tile kernel applies
    OPT_HALO_ROW, OPT_HALO_JH, OPT_HALO_JW, OPT_HALO_STACK, OPT_HALO_WIDE, OPT_HALO_PAIR, OPT_HALO_FLAT,
    OPT_HALO_NARROW, OPT_HALO_DUAL, OPT_PATCH_MATRIX, OPT_DX_PHASES, OPT_DX_COL2IM, OPT_DX_TRANSPOSE,
    OPT_DW_STACKED, OPT_DW_DIAG, OPT_DW_CW, OPT_DW_R, OPT_DW_STATIC, OPT_CONV_PROF, OPT_SM_BUDGET,
    OPT_SKINNY, OPT_HALO_DEEP, OPT_HALO_SPLITB, OPT_NVTX, OPT_DW_LANES, OPT_HALO_TAPSTACK, OPT_HALO_FLAT32,
    OPT_DW_STRIDED,     // 0 = strided deltaW on the split-K im2col kernel only
    OPT_DW_TAPGROUPS,   // 0 = a CTA always owns a whole filter row, 2 = rows of more than three taps always split
    OPT_COUNT
};
struct OptDef { const char* name; int dflt; };
static const OptDef kOptDefs[OPT_COUNT] = {
    {"CONV_TILE", 0}, {"CONV_DW", 0},
    {"HALO_ROW", 1}, {"HALO_JH", 0}, {"HALO_JW", 0}, {"HALO_STACK", 1}, {"HALO_WIDE", -1}, {"HALO_PAIR", -1}, {"HALO_FLAT", 1},
    {"HALO_NARROW", 1}, {"HALO_DUAL", 1}, {"PATCH_MATRIX", 1}, {"DX_PHASES", 1}, {"DX_COL2IM", 1}, {"DX_TRANSPOSE", 1},
    {"DW_STACKED", -1}, {"DW_DIAG", 1}, {"DW_CW", 0}, {"DW_R", 0}, {"DW_STATIC", 1}, {"CONV_PROF", 0}, {"SM_BUDGET", 0},
    {"SKINNY", 1}, {"HALO_DEEP", 1}, {"HALO_SPLITB", 0}, {"NVTX", 1}, {"DW_LANES", 0}, {"HALO_TAPSTACK", 1}, {"HALO_FLAT32", 1},
    {"DW_STRIDED", 1}, {"DW_TAPGROUPS", 1},
};
static std::atomic<int> g_opt[OPT_COUNT];
static std::once_flag g_opt_once;

static int parse_opt(int which, const char* e)
{
    if (which == OPT_CONV_TILE) {
        if (!strcmp(e, "im2col")) return 1;
        if (!strcmp(e, "halo")) return 2;
        if (!strcmp(e, "auto")) return 0;
    }
    if (which == OPT_CONV_DW && !strcmp(e, "split")) return 1;
    return atoi(e);
}
static void init_opts()
{
    for (int i = 0; i < OPT_COUNT; ++i) {
        char name[64];
        snprintf(name, sizeof(name), "ALPHA_%s", kOptDefs[i].name);
        const char* e = getenv(name);
        g_opt[i].store((e && *e) ? parse_opt(i, e) : kOptDefs[i].dflt);
    }
}
static inline int opt(Opt which)
{
    std::call_once(g_opt_once, init_opts);
    return g_opt[which].load(std::memory_order_relaxed);
}

static int env_math()
{
    const char* e = getenv("ALPHA_CONV_MATH");
    if (e && (!strcmp(e, "tf32") || !strcmp(e, "TF32"))) return ALPHA_MATH_TF32;
    return ALPHA_MATH_3XTF32;
}
static int env_algo()
{
    const char* e = getenv("ALPHA_CONV_ALGO");
    if (!e) return ALPHA_ALGO_AUTO;
    if (!strcmp(e, "tensor") || !strcmp(e, "igemm")) return ALPHA_ALGO_TENSOR;
    if (!strcmp(e, "simt")) return ALPHA_ALGO_SIMT;
    if (!strcmp(e, "winograd")) return ALPHA_ALGO_WINOGRAD;
    return ALPHA_ALGO_AUTO;
}
// Process-wide defaults of the math mode and kernel family, and the per-call values the *_ex entry
// points put in their place for the calling thread while they run.
static std::atomic<int> g_math{env_math()};
static std::atomic<int> g_algo{env_algo()};
static thread_local int t_math = -1, t_algo = -1;
static inline int cur_math() { return t_math >= 0 ? t_math : g_math.load(std::memory_order_relaxed); }
static inline int cur_algo() { return t_algo >= 0 ? t_algo : g_algo.load(std::memory_order_relaxed); }
static inline int cur_mode3x() { return cur_math() == ALPHA_MATH_3XTF32; }
struct CallOptions {
    int save_math, save_algo;
    CallOptions(int math, int algo) : save_math(t_math), save_algo(t_algo) { if (math >= 0) t_math = math; if (algo >= 0) t_algo = algo; }
    ~CallOptions() { t_math = save_math; t_algo = save_algo; }
};

// One NVTX range per operator call (option NVTX, on by default): a timeline tool attached to the process shows
// which contraction the kernels of a call belong to; without a tool a push / pop is a few nanoseconds.
struct OpRange {
    bool on;
    explicit OpRange(const char* name) : on(opt(OPT_NVTX) != 0 && !t_dry) { if (on) nvtxRangePushA(name); }
    ~OpRange() { if (on) nvtxRangePop(); }
};

// ---- per-device context ----------------------------------------------------------------------

struct DeviceCtx {
    bool init = false;
    int sm_count = 0;
    int cc_major = 0;
    int* status = nullptr;       // device status word
    unsigned long long* prof = nullptr;  // cycle counters, allocated when ALPHA_CONV_PROF=1
    // Scratch per (device, stream), one block each.  Work on one stream is ordered, so calls that
    // share a stream share its block (every call carves its requests from offset 0 again); calls on
    // different streams get different blocks and may overlap freely.  A block is library-owned and
    // grown on demand, or caller-owned (alpha_conv_set_workspace) and then never grown.
    struct Block {
        char* base = nullptr; size_t bytes = 0, used = 0;
        bool external = false;   // the caller's memory
        bool captured = false;   // handed out while its stream was being captured into a CUDA graph
    };
    std::map<cudaStream_t, Block> workspace;
    // Blocks that were outgrown.  Work enqueued earlier may still use one, so it is freed only after
    // the event recorded at retirement has completed; a block that a graph capture saw is kept until
    // alpha_conv_release_workspace() because replays of that graph still address it.
    // The event is recorded at the start of the NEXT call on the stream: the call that outgrew the block
    // may still enqueue kernels that read what it was given from it.
    struct Retired { void* ptr; size_t bytes; cudaEvent_t done; bool captured; cudaStream_t stream; };
    std::vector<Retired> retired;
    // Weight-side transforms kept across calls (alpha_conv_weight_cache): hi/lo planes, transposes.
    struct WeightKey {
        const void* W; int kind, a, b, c, d, e;
        bool operator<(const WeightKey& o) const { return std::tie(W, kind, a, b, c, d, e) < std::tie(o.W, o.kind, o.a, o.b, o.c, o.d, o.e); }
    };
    struct WeightEntry { float* ptr = nullptr; size_t bytes = 0; bool valid = false; cudaEvent_t ready = nullptr; cudaStream_t stream = nullptr; };
    std::map<WeightKey, WeightEntry> weights;
    // What each caller-owned block of prepared weights (alpha_conv_prepare_weights) holds: host-side record only.
    struct PreparedDesc { WeightKey key; size_t bytes; };
    std::map<const void*, PreparedDesc> prepared;
};
static DeviceCtx g_ctx[64];
static std::mutex g_mu;

static PFN_encodeTiled g_encodeTiled = nullptr;
static PFN_encodeIm2col g_encodeIm2col = nullptr;

static int load_driver_entry_points()
{
    if (g_encodeTiled && g_encodeIm2col) return ALPHA_OK;
    cudaDriverEntryPointQueryResult q;
    void* f = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !f)
        return fail(ALPHA_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encodeTiled = reinterpret_cast<PFN_encodeTiled>(f);
    f = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !f)
        return fail(ALPHA_E_CUDA, "cuTensorMapEncodeIm2col is not available from this driver");
    g_encodeIm2col = reinterpret_cast<PFN_encodeIm2col>(f);
    return ALPHA_OK;
}

// SMs the persistent kernels spread over: all of them, or the part alpha_conv_set_option("SM_BUDGET")
// leaves when some are to stay free for a collective that runs beside the convolutions.
static inline int sm_budget(const DeviceCtx* c);

int get_ctx(DeviceCtx** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(ALPHA_E_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx& c = g_ctx[dev];
    if (!c.init) {
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        if (prop.major != 10)
            return fail(ALPHA_E_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                        dev, prop.major, prop.minor);
        int rc = load_driver_entry_points();
        if (rc) return rc;
        e = cudaMalloc(&c.status, sizeof(int));
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMalloc(status): %s", cudaGetErrorString(e));
        cudaMemset(c.status, 0, sizeof(int));
        if (opt(OPT_CONV_PROF) > 0) {
            if (cudaMalloc(&c.prof, kProfSlots * sizeof(unsigned long long)) == cudaSuccess)
                cudaMemset(c.prof, 0, kProfSlots * sizeof(unsigned long long));
            else
                c.prof = nullptr;
        }
        c.sm_count = prop.multiProcessorCount;
        c.cc_major = prop.major;
        const int max_smem = 227 * 1024;
        cudaFuncSetAttribute(conv_igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        cudaFuncSetAttribute(conv_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        c.init = true;
    }
    *out = &c;
    return ALPHA_OK;
}

static inline int sm_budget(const DeviceCtx* c)
{
    const int b = opt(OPT_SM_BUDGET);
    return (b > 0 && b < c->sm_count) ? b : c->sm_count;
}

// ---- scratch memory ----------------------------------------------------------------------------
//
// t_caller: scratch the caller of a native handed over for this one call (the CW / deltaW_buf
// arguments of the reference's JNI signatures); requests that fit are served from it first.
static thread_local size_t t_dry_cur = 0, t_dry_peak = 0;
struct CallerScratch { char* ptr = nullptr; size_t bytes = 0, used = 0; };
static thread_local CallerScratch t_caller;

void set_caller_scratch(void* ptr, size_t bytes)
{
    t_caller.ptr = static_cast<char*>(ptr);
    t_caller.bytes = ptr ? bytes : 0;
    t_caller.used = 0;
}

static void sweep_retired(DeviceCtx* c)   // g_mu held
{
    for (size_t i = 0; i < c->retired.size();) {
        DeviceCtx::Retired& r = c->retired[i];
        if (!r.captured && r.done && cudaEventQuery(r.done) == cudaSuccess) {
            cudaEventDestroy(r.done);
            cudaFree(r.ptr);
            c->retired.erase(c->retired.begin() + i);
        } else {
            ++i;
        }
    }
    cudaGetLastError();   // cudaEventQuery reports "not ready" through the error state
}

static bool stream_is_capturing(cudaStream_t stream)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) { cudaGetLastError(); return false; }
    return st != cudaStreamCaptureStatusNone;
}

// Starts one API call on `stream`: its scratch requests are carved from the start of the block again.
static void ws_begin(DeviceCtx* c, cudaStream_t stream)
{
    if (t_dry) { t_dry_cur = t_dry_peak = 0; return; }
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = c->workspace.find(stream);
    if (it != c->workspace.end()) it->second.used = 0;
    t_caller.used = 0;
    for (DeviceCtx::Retired& r : c->retired)
        if (!r.done && !r.captured && r.stream == stream && !stream_is_capturing(stream) &&
            cudaEventCreateWithFlags(&r.done, cudaEventDisableTiming) == cudaSuccess)
            cudaEventRecord(r.done, stream);
}

static int grow_block(DeviceCtx* c, cudaStream_t stream, DeviceCtx::Block& b, size_t need)   // g_mu held
{
    if (b.external)
        return fail(ALPHA_E_NOSCRATCH, "the workspace given by alpha_conv_set_workspace holds %zu bytes, this call needs %zu "
                    "(alpha_conv_workspace_bytes tells in advance)", b.bytes, need);
    if (stream_is_capturing(stream))
        return fail(ALPHA_E_CAPTURE, "the call needs %zu bytes of scratch, the stream's block holds %zu, and the stream is being "
                    "captured: run the step once eagerly or call alpha_conv_reserve_workspace before capturing", need, b.bytes);
    sweep_retired(c);
    const size_t want = need + (need >> 2);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ALPHA_E_CUDA, "cudaMalloc(workspace %zu B): %s", want, cudaGetErrorString(e)); }
    if (b.base) {
        c->retired.push_back(DeviceCtx::Retired{b.base, b.bytes, nullptr, b.captured, stream});
    }
    b.base = static_cast<char*>(p); b.bytes = want; b.captured = false;
    return ALPHA_OK;
}

// `bytes` of scratch for the current call on `stream`, valid until the work enqueued by this call
// has run.  Requests of one call do not overlap each other.
static int get_workspace(DeviceCtx* c, cudaStream_t stream, size_t bytes, float** out, int = 0)
{
    bytes = (bytes + 255) & ~static_cast<size_t>(255);
    if (t_dry) {
        t_dry_cur += bytes;
        if (t_dry_cur > t_dry_peak) t_dry_peak = t_dry_cur;
        *out = reinterpret_cast<float*>(static_cast<uintptr_t>(1) << 30);   // aligned placeholder, never dereferenced
        return ALPHA_OK;
    }
    if (t_caller.ptr && t_caller.used + bytes <= t_caller.bytes) {
        *out = reinterpret_cast<float*>(t_caller.ptr + t_caller.used);
        t_caller.used += bytes;
        return ALPHA_OK;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx::Block& b = c->workspace[stream];
    if (b.used + bytes > b.bytes) {
        int rc = grow_block(c, stream, b, b.used + bytes);
        if (rc) return rc;
    }
    if (!b.captured && !b.external && stream_is_capturing(stream)) b.captured = true;
    *out = reinterpret_cast<float*>(b.base + b.used);
    b.used += bytes;
    return ALPHA_OK;
}

// A loop whose iterations each need scratch that is dead once the iteration's kernels have been
// enqueued (they all run on one stream, in order) takes a mark before the loop body and rewinds to
// it afterwards, so that the iterations reuse the same bytes.
struct WsMark { size_t block_used, caller_used, dry_cur; };
static WsMark ws_mark(DeviceCtx* c, cudaStream_t stream)
{
    WsMark m{0, t_caller.used, t_dry_cur};
    if (!t_dry) {
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = c->workspace.find(stream);
        if (it != c->workspace.end()) m.block_used = it->second.used;
    }
    return m;
}
static void ws_rewind(DeviceCtx* c, cudaStream_t stream, const WsMark& m)
{
    t_caller.used = m.caller_used;
    t_dry_cur = m.dry_cur;
    if (t_dry) return;
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = c->workspace.find(stream);
    if (it != c->workspace.end()) it->second.used = m.block_used;
}

static int check_launch(const char* what);

// ---- weight-side transforms --------------------------------------------------------------------
//
// The forward kernels in 3xTF32 need the lo plane of W, deltaX needs W transposed (and rotated, or cut
// into stride phases) in hi and lo planes.  Weights change only when the optimizer updates them
// (the reference's contract: Tensor.java:208-221, Engine.java:341-350), so with the weight cache on
// (alpha_conv_weight_cache) a transform is computed once and kept in library-owned memory until
// alpha_conv_weights_updated() names its source tensor; with the cache off it is recomputed by
// every call into that call's scratch.
enum { WK_FWD_LO = 1, WK_DX_S1 = 2, WK_DX_PHASES = 3, WK_DX_COL2IM = 4 };
static std::atomic<int> g_weight_cache{0};

// A forward native that was handed the caller's CW block finds the lo plane kernel_remode left there.
struct PreparedLo { const float* W = nullptr; const float* lo = nullptr; };
static thread_local PreparedLo t_prepared_lo;
void set_prepared_lo(const float* W, const float* lo) { t_prepared_lo.W = W; t_prepared_lo.lo = lo; }

// Memory for one transform of `bytes`; *fresh says whether the caller still has to compute it (then
// it calls weight_planes_ready after enqueuing the kernels that do).
// Caller-owned prepared weights (alpha_conv_prepare_weights / *_prepared): for the duration of one call the
// transform of tensor W lives in the caller's block.  mode 1 = compute it there (the call runs "dry": only
// the transform is launched), 2 = it is there already, 3 = only report its size.
struct PreparedHint { const float* W = nullptr; float* ptr = nullptr; size_t bytes = 0; int mode = 0; size_t need = 0; bool seen = false; };
static thread_local PreparedHint t_prep;
static inline bool transforms_run() { return !t_dry || t_prep.mode == 1; }

static int weight_planes(DeviceCtx* c, cudaStream_t stream, const DeviceCtx::WeightKey& key, size_t bytes, float** out, bool* fresh)
{
    *fresh = true;
    if (t_prep.mode && t_prep.W == key.W) {
        t_prep.need = bytes; t_prep.seen = true;
        if (t_prep.mode == 3) { *out = reinterpret_cast<float*>(static_cast<uintptr_t>(1) << 30); return ALPHA_OK; }
        if (bytes > t_prep.bytes)
            return fail(ALPHA_E_NOSCRATCH, "the prepared-weights block holds %zu bytes, this layer's transform needs %zu "
                        "(alpha_conv_prepared_weights_bytes tells in advance)", t_prep.bytes, bytes);
        std::lock_guard<std::mutex> lock(g_mu);
        if (t_prep.mode == 1) {
            c->prepared[t_prep.ptr] = DeviceCtx::PreparedDesc{key, bytes};
        } else {
            auto it = c->prepared.find(t_prep.ptr);
            if (it == c->prepared.end() || it->second.key < key || key < it->second.key)
                return fail(ALPHA_E_ARG, "the prepared-weights block was not made by alpha_conv_prepare_weights for this tensor, "
                            "shape, operator and math mode");
            *fresh = false;
        }
        *out = t_prep.ptr;
        return ALPHA_OK;
    }
    if (t_dry || !g_weight_cache.load(std::memory_order_relaxed)) return get_workspace(c, stream, bytes, out);
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx::WeightEntry& e = c->weights[key];
    if (e.valid && e.bytes >= bytes) {
        // computed by an earlier call; a different stream waits for the kernels that wrote it
        if (e.stream != stream && e.ready && cudaEventQuery(e.ready) != cudaSuccess) {
            cudaGetLastError();
            cudaStreamWaitEvent(stream, e.ready, 0);
        }
        *out = e.ptr; *fresh = false;
        return ALPHA_OK;
    }
    if (e.bytes < bytes) {
        if (stream_is_capturing(stream))
            return fail(ALPHA_E_CAPTURE, "the weight cache has no entry for this tensor yet and the stream is being captured: "
                        "run the layer once eagerly before capturing");
        if (e.ptr) c->retired.push_back(DeviceCtx::Retired{e.ptr, e.bytes, nullptr, false, e.stream});
        void* p = nullptr;
        cudaError_t err = cudaMalloc(&p, bytes);
        if (err != cudaSuccess) { cudaGetLastError(); e = DeviceCtx::WeightEntry{}; return fail(ALPHA_E_CUDA, "cudaMalloc(weight cache %zu B): %s", bytes, cudaGetErrorString(err)); }
        e.ptr = static_cast<float*>(p); e.bytes = bytes;
    }
    e.valid = false; e.stream = stream;
    *out = e.ptr;
    return ALPHA_OK;
}
static void weight_planes_ready(DeviceCtx* c, cudaStream_t stream, const DeviceCtx::WeightKey& key)
{
    if (t_dry || !g_weight_cache.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = c->weights.find(key);
    if (it == c->weights.end()) return;
    DeviceCtx::WeightEntry& e = it->second;
    if (!e.ready && cudaEventCreateWithFlags(&e.ready, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); e.ready = nullptr; }
    if (e.ready && !stream_is_capturing(stream)) cudaEventRecord(e.ready, stream);
    e.valid = true;
}

// 3xTF32 forward: W serves as its own hi plane, this returns the lo plane.
static int forward_lo_plane(DeviceCtx* c, cudaStream_t stream, const float* W, size_t nW, const float** lo)
{
    if (t_prepared_lo.W == W && t_prepared_lo.lo) { *lo = t_prepared_lo.lo; return ALPHA_OK; }
    float* ws = nullptr;
    bool fresh = true;
    const DeviceCtx::WeightKey key{W, WK_FWD_LO, (int)(nW & 0x7fffffff), 0, 0, 0, 0};
    int rc = weight_planes(c, stream, key, nW * sizeof(float), &ws, &fresh);
    if (rc) return rc;
    if (fresh) {
        const size_t n4 = nW / 4;
        size_t blocks = (n4 + 255) / 256;
        if (blocks > (size_t)c->sm_count * 8) blocks = (size_t)c->sm_count * 8;
        if (transforms_run()) split_lo_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(W), reinterpret_cast<float4*>(ws), n4);
        note_launch("split_w");
        rc = check_launch("split_lo_kernel");
        if (rc) return rc;
        weight_planes_ready(c, stream, key);
    }
    *lo = ws;
    return ALPHA_OK;
}

// lo = lo plane of W (n floats) for alpha_Cuda_conv3D_kernel_remode: the one thing the forward natives need prepared.
int launch_split_lo(cudaStream_t stream, const float* W, float* lo, size_t n)
{
    int sms = 148;
    const size_t n4 = n / 4;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > (size_t)sms * 8) blocks = (size_t)sms * 8;
    if (blocks < 1) blocks = 1;
    split_lo_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(W), reinterpret_cast<float4*>(lo), n4);
    note_launch("split_w");
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "split_lo_kernel launch failed: %s", cudaGetErrorString(e));
    return ALPHA_OK;
}

// ---- tensor maps -----------------------------------------------------------------------------

static CUtensorMapSwizzle swizzle_for_row_bytes(int row_bytes)
{
    return row_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B
           : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                             : CU_TENSOR_MAP_SWIZZLE_32B;
}
static uint32_t desc_layout_for_row_bytes(int row_bytes)
{
    return row_bytes >= 128 ? kSwizzle128B : row_bytes == 64 ? kSwizzle64B : kSwizzle32B;
}

// NHWC activation tensor [N,H,W,C] as an im2col-mode map over (C, W, H, N).
// Base pixels run over w in [-pad_w, W + pad_w - (FW-1)) with step sw, likewise for h.
static int make_im2col_map(CUtensorMap* m, const float* base, int N, int H, int W, int C, int FH,
                           int FW, int sh, int sw, int pad_h, int pad_w, int channels, int pixels,
                           CUtensorMapSwizzle swz)
{
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
    int lower[2] = {-pad_w, -pad_h};
    int upper[2] = {pad_w - (FW - 1), pad_h - (FH - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
    CUresult r = g_encodeIm2col(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims,
                                strides, lower, upper, (cuuint32_t)channels, (cuuint32_t)pixels, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    // Drivers up to CUDA 13.1 set a descriptor bit for im2col maps that must be clear when the
    // tensor is smaller than 128 KiB (the same correction CUTLASS applies after encoding).
    int drv = 0;
    if (r == CUDA_SUCCESS && cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
        (size_t)N * H * W * C * 4 < 131072)
        reinterpret_cast<uint64_t*>(m)[1] &= ~(1ull << 21);
    if (r != CUDA_SUCCESS)
        return fail(ALPHA_E_CUDA,
                    "cuTensorMapEncodeIm2col failed (%d): dims C=%d W=%d H=%d N=%d corners [%d,%d]/[%d,%d] "
                    "channels=%d pixels=%d strides %d,%d",
                    (int)r, C, W, H, N, lower[0], lower[1], upper[0], upper[1], channels, pixels, sw, sh);
    return ALPHA_OK;
}

static int make_tiled_map(CUtensorMap* m, const float* base, int rank, const cuuint64_t* dims,
                          const cuuint64_t* strides_bytes, const cuuint32_t* box, CUtensorMapSwizzle swz)
{
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = g_encodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank,
                               const_cast<float*>(base), dims, strides_bytes, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ALPHA_E_CUDA, "cuTensorMapEncodeTiled failed (%d), rank %d box0 %u", (int)r, rank, box[0]);
    return ALPHA_OK;
}

// ---- argument checks -------------------------------------------------------------------------

static int check_shape(const AlphaConvShape* s, const void* a, const void* b, const void* c)
{
    if (!s || !a || !b || !c) return fail(ALPHA_E_ARG, "null shape or tensor pointer");
    if (s->N <= 0 || s->IH <= 0 || s->IW <= 0 || s->IC <= 0 || s->OC <= 0 || s->FH <= 0 || s->FW <= 0 ||
        s->OH <= 0 || s->OW <= 0 || s->sh <= 0 || s->sw <= 0 || s->ph < 0 || s->pw < 0)
        return fail(ALPHA_E_ARG, "non-positive dimension in conv shape");
    if ((s->IC & 3) || (s->OC & 3))
        return fail(ALPHA_E_ARG, "IC=%d and OC=%d must be multiples of 4 (padded channel stride)", s->IC, s->OC);
    if ((s->OH - 1) * s->sh - s->ph + s->FH > s->IH + s->ph || (s->OW - 1) * s->sw - s->pw + s->FW > s->IW + s->pw)
        return fail(ALPHA_E_ARG, "OH/OW=%d/%d do not fit IH/IW=%d/%d with this filter, stride and padding",
                    s->OH, s->OW, s->IH, s->IW);
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15)
        return fail(ALPHA_E_ARG, "tensor pointers must be 16-byte aligned");
    const long long lim = 2147483647LL;
    if ((long long)s->N * s->IH * s->IW * s->IC > lim || (long long)s->N * s->OH * s->OW * s->OC > lim ||
        (long long)s->OC * s->FH * s->FW * s->IC > lim)
        return fail(ALPHA_E_ARG, "tensor has more than 2^31-1 elements");
    return ALPHA_OK;
}

static int pick_kc(int channels)
{
    return (channels % 32 == 0) ? 32 : (channels % 16 == 0) ? 16 : (channels % 8 == 0) ? 8 : 0;
}

static uint32_t pow2_cols(int n)
{
    uint32_t c = 32;
    while ((int)c < n) c <<= 1;
    return c;
}

static int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return ALPHA_OK;
}

static int simt_grid(size_t total, int sm_count)
{
    size_t blocks = (total + 255) / 256;
    size_t cap = (size_t)sm_count * 32;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

static ConvShape to_dev_shape(const AlphaConvShape* s)
{
    ConvShape d{s->N, s->IH, s->IW, s->IC, s->OC, s->FH, s->FW, s->OH, s->OW, s->sh, s->sw, s->ph, s->pw};
    return d;
}

// ---- implicit GEMM launch shared by forward and stride-1 deltaX -----------------------------------

struct IgemmPlan {
    // activation tensor seen by the im2col map
    const float* act; int aN, aH, aW, aC;
    int FH, FW, sh, sw, pad_h, pad_w;
    // output
    float* out; int oH, oW, ncols;
    const float* W; int wOC, wIC;   // W[wOC][FH*FW][wIC]
    const float* bias;
    int act_on = 0; float act_k = 0.f;   // LeakyReLU after the bias (forward only)
    bool b_mn, flip;
    int kdim;                        // reduction channels per tap
    const float* W_lo = nullptr;     // when set, W and W_lo already are the hi and lo TF32 planes
    // output element (n, oh, ow, c) lives at out[((n * oNH + oh * oSH) * oNW + ow * oSW) * ncols + c]:
    // a stride phase of deltaX writes every oSH-th row and oSW-th column of an oNH x oNW image
    int oSH = 1, oSW = 1, oNH = 0, oNW = 0;
    bool force = false;              // take the halo kernel even when few tile pixels are real
    int w_img_rows = 0;              // > 0: image n uses rows [n * w_img_rows, ...) of W (batched matrix products)
};

static int launch_igemm(DeviceCtx* c, const IgemmPlan& pl, int mode3x, cudaStream_t stream)
{
    const int KC = pick_kc(pl.kdim);
    IgemmParams p{};
    p.out = pl.out; p.bias = pl.bias; p.act_on = pl.act_on; p.act_k = pl.act_k; p.status = c->status;
    p.M_total = pl.aN * pl.oH * pl.oW;
    p.Ncols = pl.ncols; p.ldo = pl.ncols;
    p.OHo = pl.oH; p.OWo = pl.oW;
    p.sh = pl.sh; p.sw = pl.sw; p.ph = pl.pad_h; p.pw = pl.pad_w;
    p.FH = pl.FH; p.FW = pl.FW;
    p.KC = KC; p.kchunks = pl.kdim / KC;
    p.mode3x = mode3x; p.b_mn = pl.b_mn; p.flip = pl.flip;
    const int gran = pl.b_mn ? 32 : 16;
    int BN = ((pl.ncols + gran - 1) / gran) * gran;
    if (BN > 256) BN = (pl.ncols % 256 == 0 || pl.ncols > 512) ? 256 : 128;
    p.BN = BN;
    p.tmem_cols = pow2_cols(BN);
    p.idesc = make_idesc_tf32(kBM, BN, false, pl.b_mn);
    p.a_bytes = kBM * KC * 4;
    p.b_tx = pl.b_mn ? (BN / 32) * KC * 128 : BN * KC * 4;
    p.b_bytes = (p.b_tx + 1023) & ~1023u;
    p.swz = desc_layout_for_row_bytes(KC * 4);
    const uint32_t stage = (p.a_bytes + p.b_bytes) * (mode3x ? 2 : 1);
    int stages = (int)((100u * 1024) / stage);      // aim at two resident CTAs per SM
    if (stages < 3) stages = (int)((200u * 1024) / stage);
    if (stages > 6) stages = 6;
    const int num_it = pl.FH * pl.FW * p.kchunks;
    if (stages > num_it) stages = num_it;
    if (stages < 1) return fail(ALPHA_E_ARG, "tile of %u bytes per stage does not fit shared memory", stage);
    p.stages = stages;
    const size_t smem = (size_t)stages * stage + (3 * stages + 2) * 8 + 1024;

    CUtensorMap tmA, tmB;
    int rc = make_im2col_map(&tmA, pl.act, pl.aN, pl.aH, pl.aW, pl.aC, pl.FH, pl.FW, pl.sh, pl.sw,
                             pl.pad_h, pl.pad_w, KC, kBM, swizzle_for_row_bytes(KC * 4));
    if (rc) return rc;
    cuuint64_t wd[3] = {(cuuint64_t)pl.wIC, (cuuint64_t)pl.FH * pl.FW, (cuuint64_t)pl.wOC};
    cuuint64_t ws[2] = {(cuuint64_t)pl.wIC * 4, (cuuint64_t)pl.FH * pl.FW * pl.wIC * 4};
    if (!pl.b_mn) {
        cuuint32_t box[3] = {(cuuint32_t)KC, 1, (cuuint32_t)BN};
        rc = make_tiled_map(&tmB, pl.W, 3, wd, ws, box, swizzle_for_row_bytes(KC * 4));
    } else {
        cuuint32_t box[3] = {32, 1, (cuuint32_t)KC};
        rc = make_tiled_map(&tmB, pl.W, 3, wd, ws, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    }
    if (rc) return rc;

    dim3 grid((p.M_total + kBM - 1) / kBM, (pl.ncols + BN - 1) / BN, 1);
    if (!t_dry) conv_igemm_kernel<<<grid, kIgemmThreads, smem, stream>>>(tmA, tmB, p);
    note_launch("igemm");
    return check_launch("conv_igemm_kernel");
}

// ---- halo-tile kernel (stride 1): plan and launch -------------------------------------------------

static inline int env_tile_mode() { return opt(OPT_CONV_TILE); }

struct HaloChoice {
    bool valid = false;
    int JH = 1, JW = 1, npb = 1, sb = 2, acc_bufs = 1, NI = 1;
    bool row = false, stat = false, wide = false;
    bool flat = false;   // accumulators of 4 rows x 32 patch columns, one patch each (JH * JW of them per macro tile)
    double cost = 0, eff = 0;
};

// Picks the macro-tile shape.  Cost = estimated SM cycles per useful output pixel: the larger of the
// MMA issue time and the L2->SM transfer time, divided by the fraction of tile pixels that are
// real, with small penalties for single-buffered patches / accumulators.
// The row-staged specialisations that exist (FW, JH, JW); everything else runs the generic form.
static bool halo_has_row_kernel(int FW, int JH, int JW)
{
    if (FW != 1 && FW != 2 && FW != 3 && FW != 5) return false;
    return (JH == 1 && (JW == 1 || JW == 2 || JW == 4)) || (JH == 2 && (JW == 1 || JW == 2));
}

struct HaloLaunch {
    int grid;
    size_t smem;
    cudaStream_t stream;
    const CUtensorMap *tmA, *tmB, *tmBlo, *tmO;
    const HaloParams* p;
};

template <int FW_T, int JH_T, int JW_T, bool ROW_T, bool FLAT_T = false>
static void halo_launch_one(const HaloLaunch& L)
{
    static bool attr_done = false;  // per instantiation; the attribute is per function, any device
    if (!attr_done) {
        cudaFuncSetAttribute(conv_halo_kernel<FW_T, JH_T, JW_T, ROW_T, FLAT_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr_done = true;
    }
    if (!t_dry) conv_halo_kernel<FW_T, JH_T, JW_T, ROW_T, FLAT_T><<<L.grid, kHaloThreads2, L.smem, L.stream>>>(*L.tmA, *L.tmB, *L.tmBlo, *L.tmO, *L.p);
}

template <int FW_T>
static void halo_launch_fw(const HaloLaunch& L, int JH, int JW, bool row)
{
#define HALO_J(JH_, JW_) do { if (row) halo_launch_one<FW_T, JH_, JW_, true>(L); else halo_launch_one<FW_T, JH_, JW_, false>(L); } while (0)
    if (JH == 1 && JW == 1) HALO_J(1, 1);
    else if (JH == 1 && JW == 2) HALO_J(1, 2);
    else if (JH == 1 && JW == 4) HALO_J(1, 4);
    else if (JH == 2 && JW == 1) HALO_J(2, 1);
    else HALO_J(2, 2);
#undef HALO_J
}

// Split-K parts for a launch of `tiles` macro tiles whose reduction has `kchunks` chunks of `taps` W-tile
// stages each: 1 unless the tiles cover less than half of the SMs and the reduction is long enough.
static int halo_ksplit(const IgemmPlan& pl, long long tiles, int kchunks, int sm_count)
{
    const bool dense_out = pl.oSH == 1 && pl.oSW == 1 && pl.oNH == 0 && pl.oNW == 0;
    const int taps = pl.FH * pl.FW;
    if (!dense_out || pl.w_img_rows || !opt(OPT_SKINNY) || kchunks < 2 || 2 * tiles > sm_count || (long long)kchunks * taps < 16) return 1;
    int ksplit = (int)(sm_count / tiles);
    if (ksplit > 16) ksplit = 16;
    if (ksplit > kchunks) ksplit = kchunks;
    // every part gets at least four W-tile stages to amortise its prologue and epilogue
    while (ksplit > 1 && (long long)((kchunks + ksplit - 1) / ksplit) * taps < 4) --ksplit;
    const int cps = (kchunks + ksplit - 1) / ksplit;
    return (kchunks + cps - 1) / cps;
}

static HaloChoice plan_halo(const IgemmPlan& pl, int BN, int mode3x, int b_mn, int sm_count)
{
    HaloChoice best;
    const int taps = pl.FH * pl.FW, kchunks = pl.kdim / 32;
    const int planes = mode3x ? 2 : 1;
    const uint32_t b_tx = b_mn ? (BN / 32) * 4096 : BN * 128;
    const uint32_t b_tile = ((b_tx + 1023) & ~1023u) * planes;
    const bool allow_row = opt(OPT_HALO_ROW) != 0;
    const int force_jh = opt(OPT_HALO_JH), force_jw = opt(OPT_HALO_JW);
    const size_t smem_cap = 226 * 1024;
    // small images: NI images stacked in one accumulator, each in a slot of SG = OH + FH - 1 rows
    const int SG = pl.oH + pl.FH - 1;
    int ni_max = 1;
    if (SG <= 16 && opt(OPT_HALO_STACK) && !pl.w_img_rows) ni_max = 1 + (16 - pl.oH) / SG;
    // 3xTF32 with BN <= 128: the wide form (hi x [hi | lo] in one MMA of 2*BN columns, then lo x hi) needs
    // max(BN, 59) + max(BN / 2, 59) clocks per step instead of 3 * max(BN / 2, 59) and reads the A
    // operand twice instead of three times, at twice the tensor-memory columns per accumulator
    const int wide_env = opt(OPT_HALO_WIDE);
    const int wide_lo = (mode3x && BN <= 128 && wide_env != 0) ? (wide_env == 1 ? 1 : 0) : 0;
    const int wide_hi = (mode3x && BN <= 128 && wide_env != 0) ? 1 : 0;
    for (int wide = wide_lo; wide <= wide_hi; ++wide)
    for (int NI = 1; NI <= ni_max; NI += (ni_max > 1 ? ni_max - 1 : 1))
    for (int JH = 1; JH <= 2; ++JH)
        for (int JW = 1; JW <= 4; ++JW) {
            const int accw = wide ? 2 * BN : BN;
            if (NI > 1 && (JH != 1 || JW != 1)) continue;
            if (force_jh && JH != force_jh) continue;
            if (force_jw && JW != force_jw) continue;
            const int J = JH * JW;
            if (J * accw > 512) continue;
            const int PH = NI > 1 ? NI * SG : 16 * JH + pl.FH - 1, PW = 8 * JW + pl.FW - 1;
            if (PH > 256 || PW > 256) continue;
            const uint32_t patch_stride = (((uint32_t)PH * PW * 128 + 1023) & ~1023u) * planes;
            const bool stat = allow_row && !b_mn && halo_has_row_kernel(pl.FW, JH, JW);  // a static specialisation exists (K-major W only)
            bool row = stat;
            uint32_t b_stride = b_tile * (row ? pl.FW : 1);
            if (row && (size_t)patch_stride + 2 * (size_t)b_stride + 32768 + 1536 > smem_cap) { row = false; b_stride = b_tile; }
            const int max_sb = row ? pl.FH * 2 : 8;
            int npb = 2, sb = row ? 3 : 4;
            auto need = [&](int a, int b) { return (size_t)a * patch_stride + (size_t)b * b_stride + 32768 + 512 + 1024; };
            while (need(npb, sb) > smem_cap && sb > 2) --sb;
            if (need(npb, sb) > smem_cap) { npb = 1; sb = 4; while (need(npb, sb) > smem_cap && sb > 2) --sb; }
            if (need(npb, sb) > smem_cap) continue;
            while (sb < max_sb && need(npb, sb + 1) <= smem_cap && sb < taps) ++sb;
            if (taps == 1 && opt(OPT_HALO_DEEP)) {
                // a 1x1 product (also every patch-matrix form): one chunk is four K steps of work, far less
                // than the latency of the loads that feed it, so the rings go as deep as shared memory allows
                for (int cand = 6; cand > npb; --cand)
                    if (need(cand, cand) <= smem_cap) { npb = cand; sb = cand; break; }
                while (need(npb, sb + 1) <= smem_cap && sb < 8) ++sb;
            }
            const int acc_bufs = (2 * J * accw <= 512) ? 2 : 1;
            const int rbk = NI > 1 ? 1 : (pl.oH + 16 * JH - 1) / (16 * JH), cbk = (pl.oW + 8 * JW - 1) / (8 * JW);
            const double eff = NI > 1 ? (double)NI * pl.oH * pl.oW / (128.0 * cbk)
                                      : (double)pl.oH * pl.oW / ((double)rbk * 16 * JH * cbk * 8 * JW);
            // cycles per macro tile: one tcgen05.mma of this shape takes max(N/2, 59) clocks
            auto clk = [](double n) { return n / 2.0 > 59.0 ? n / 2.0 : 59.0; };
            const double step_clk = wide ? clk(2.0 * BN) + clk(BN) : (mode3x ? 3 : 1) * clk(BN);
            const double t_mma = (double)taps * kchunks * 4 * J * step_clk;
            // shared-memory traffic per macro tile at 128 B/clk: the operands every MMA reads (4 KB of A,
            // 32 B per column of B), what the TMA writes, the lo planes the split warps read and write,
            // and the epilogue's staging.  A tcgen05.mma of 128 columns saturates this by itself.
            const double step_bytes = wide ? (4096.0 + 64.0 * BN) + (4096.0 + 32.0 * BN)
                                           : (mode3x ? 3 : 1) * (4096.0 + 32.0 * BN);
            const double tma_bytes = (double)kchunks * ((double)PH * PW * 128 + (double)taps * b_tx * planes);
            const double smem_bytes = (double)taps * kchunks * 4 * J * step_bytes + tma_bytes +
                                      (mode3x ? 2.0 * kchunks * PH * PW * 128 : 0.0) + 2.0 * 128 * J * BN * 4;
            const double t_smem = smem_bytes / 128.0;
            // W tiles are read by every CTA at about the same time and cost about half of private bytes
            const double bytes = (double)kchunks * ((double)PH * PW * 128 + 0.5 * taps * b_tx * planes) + 128.0 * J * BN * 4;
            const double t_l2 = bytes / 28.0;  // ~28 B/clk/SM between L2 and an SM when all SMs pull
            double t = t_mma + 1500.0;         // fixed per-tile overhead of the issue loop
            if (t_smem + 500.0 > t) t = t_smem + 500.0;
            if (t_l2 > t) t = t_l2;
            if (npb == 1) t *= 1.25;
            if (acc_bufs == 1) t *= 1.15;
            if (!stat) t *= 1.3; else if (!row) t *= 1.05;
            // whole-launch cost: the busiest persistent CTA walks ceil(tiles / SMs) macro tiles
            const long long n_macro = (long long)((pl.ncols + BN - 1) / BN) * ((pl.aN + NI - 1) / NI) * rbk * cbk;
            double cost = t * (double)((n_macro + sm_count - 1) / sm_count);
            // few tiles: the launch splits the reduction over idle SMs (halo_ksplit), so a wide tile that
            // moves fewer bytes per FLOP no longer costs parallelism
            const int ks = halo_ksplit(pl, n_macro, kchunks, sm_count);
            if (ks > 1) cost = t / ks + 4000.0;
            if (!best.valid || cost < best.cost) {
                best.valid = true; best.JH = JH; best.JW = JW; best.npb = npb; best.sb = sb;
                best.acc_bufs = acc_bufs; best.cost = cost; best.eff = eff; best.row = row; best.stat = stat; best.NI = NI; best.wide = wide != 0;
            }
        }
    // Flat tiles (images at most 30 pixels wide, 3x3 filters, K-major W): two accumulators of 4 rows x 32 patch
    // columns per W tile, each with its own patch, taken from the list of all four-row blocks of the batch - a
    // 28 x 28 image is seven of them, which 16 x 8 tiles cover with 0.77 of their lanes and these with 0.875.
    if (opt(OPT_HALO_FLAT32) && allow_row && !b_mn && pl.FW == 3 && pl.oW + pl.FW - 1 <= 32 && !pl.w_img_rows &&
        pl.oSH == 1 && pl.oSW == 1 && pl.oNH == 0 && pl.oNW == 0 && 2 * 2 * BN <= 512 && !force_jh && !force_jw) {
        const int J = 2, wide = (mode3x && BN <= 128 && wide_env != 0) ? 1 : 0;
        const int accw = wide ? 2 * BN : BN;
        const int PHf = 4 + pl.FH - 1;
        const uint32_t patch_stride = (uint32_t)J * PHf * 32 * 128 * planes;
        bool row = true;
        uint32_t b_stride = b_tile * pl.FW;
        if ((size_t)patch_stride + 2 * (size_t)b_stride + 32768 + 1536 > smem_cap) { row = false; b_stride = b_tile; }
        const int max_sb = row ? pl.FH * 2 : 8;
        int npb = 2, sb = row ? 3 : 4;
        auto need = [&](int a, int b) { return (size_t)a * patch_stride + (size_t)b * b_stride + 32768 + 512 + 1024; };
        while (need(npb, sb) > smem_cap && sb > 2) --sb;
        if (need(npb, sb) > smem_cap) { npb = 1; sb = 4; while (need(npb, sb) > smem_cap && sb > 2) --sb; }
        if (need(npb, sb) <= smem_cap && J * accw * 1 <= 512) {
            while (sb < max_sb && need(npb, sb + 1) <= smem_cap && sb < taps) ++sb;
            const int acc_bufs = (2 * J * accw <= 512) ? 2 : 1;
            const long long rb4 = (pl.oH + 3) / 4, blocks = (long long)pl.aN * rb4, macro = (blocks + J - 1) / J;
            const double eff = (double)pl.aN * pl.oH * pl.oW / ((double)macro * J * 128.0);
            auto clk = [](double n) { return n / 2.0 > 59.0 ? n / 2.0 : 59.0; };
            const double step_clk = wide ? clk(2.0 * BN) + clk(BN) : (mode3x ? 3 : 1) * clk(BN);
            const double t_mma = (double)taps * kchunks * 4 * J * step_clk;
            const double step_bytes = wide ? (4096.0 + 64.0 * BN) + (4096.0 + 32.0 * BN) : (mode3x ? 3 : 1) * (4096.0 + 32.0 * BN);
            const double patch_b = (double)J * PHf * 32 * 128;
            const double tma_bytes = (double)kchunks * (patch_b + (double)taps * b_tx * planes);
            const double smem_bytes = (double)taps * kchunks * 4 * J * step_bytes + tma_bytes + (mode3x ? 2.0 * kchunks * patch_b : 0.0) +
                                      2.0 * 128 * J * BN * 4;
            const double t_smem = smem_bytes / 128.0;
            const double bytes = (double)kchunks * (patch_b + 0.5 * taps * b_tx * planes) + 128.0 * J * BN * 4;
            double t = t_mma + 1500.0;
            if (t_smem + 500.0 > t) t = t_smem + 500.0;
            if (bytes / 28.0 > t) t = bytes / 28.0;
            if (npb == 1) t *= 1.25;
            if (acc_bufs == 1) t *= 1.15;
            if (!row) t *= 1.05;
            const long long n_macro = (long long)((pl.ncols + BN - 1) / BN) * macro;
            const double cost = t * (double)((n_macro + sm_count - 1) / sm_count);
            const bool forced = opt(OPT_HALO_FLAT32) == 2;
            // (few macro tiles: the 16 x 8 forms can split the reduction over idle SMs, this one cannot)
            if (forced || (2 * n_macro > sm_count && (!best.valid || cost < 0.97 * best.cost))) {
                best = HaloChoice{};
                best.valid = true; best.JH = 2; best.JW = 1; best.npb = npb; best.sb = sb; best.acc_bufs = acc_bufs;
                best.cost = cost; best.eff = eff; best.row = row; best.stat = true; best.NI = 1; best.wide = wide != 0; best.flat = true;
            }
        }
    }
    return best;
}

// ---- halo kernel on CTA pairs ----------------------------------------------------------------------
template <int FW_T, bool ROW_T, bool FLAT_T = false>
static void halo_pair_launch_one(const HaloLaunch& L)
{
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(conv_halo_pair_kernel<FW_T, ROW_T, FLAT_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr_done = true;
    }
    if (!t_dry) conv_halo_pair_kernel<FW_T, ROW_T, FLAT_T><<<L.grid, kHaloThreads, L.smem, L.stream>>>(*L.tmA, *L.tmB, *L.tmBlo, *L.tmO, *L.p);
}

// One 16 x 8 pixel accumulator per CTA, two CTAs per MMA.  Returns 1 when the shape does not fit.
static int launch_halo_pair(DeviceCtx* c, const IgemmPlan& pl, int mode3x, cudaStream_t stream)
{
    if (pl.FW != 3 || pl.sh != 1 || pl.sw != 1 || pl.kdim % 32 != 0 || pl.b_mn) return 1;
    int BN = ((pl.ncols + 15) / 16) * 16;
    // wide 3xTF32 needs 2 * BN <= 256 columns per MMA; ALPHA_HALO_PAIR=2 takes three MMAs of BN <= 256 instead
    const int pair_env = opt(OPT_HALO_PAIR);
    const bool three = mode3x && pair_env != 1;
    // the side-column form of the three-MMA mode needs 2 * BN columns per accumulator, twice
    const bool side3 = three && pair_env != 2;
    // side columns with BN = 256 fill all 512 tensor-memory columns with ONE accumulator set, so the
    // epilogue no longer overlaps the next tile; that pays once the reduction is long (7x7x512:
    // 0.320 -> 0.296 ms, half as many patch loads), not before (14x14x256: 0.281 -> 0.314 ms)
    const bool side_wide = side3 && ((pl.ncols % 256 == 0 && pl.kdim >= 512) || pair_env == 4);
    const int bn_max = (mode3x && !(three && !side3) && !side_wide) ? 128 : 256;
    if (BN > bn_max) {
        if (pl.ncols % bn_max == 0) BN = bn_max;
        else if (pl.ncols % (bn_max / 2) == 0) BN = bn_max / 2;
        else return 1;
    }
    const int SG = pl.oH + pl.FH - 1;
    int NI = 1;
    if (SG <= 16 && opt(OPT_HALO_STACK)) NI = 1 + (16 - pl.oH) / SG;
    HaloParams p{};
    p.out = pl.out; p.bias = pl.bias; p.act_on = pl.act_on; p.act_k = pl.act_k; p.status = c->status; p.prof = c->prof;
    p.N = pl.aN; p.OH = pl.oH; p.OW = pl.oW;
    p.Ncols = pl.ncols; p.ldo = pl.ncols;
    p.FH = pl.FH; p.FW = pl.FW; p.pad_h = pl.pad_h; p.pad_w = pl.pad_w;
    p.kchunks = pl.kdim / 32;
    p.BN = BN; p.n_tiles = (pl.ncols + BN - 1) / BN;
    p.JH = 1; p.JW = 1; p.NI = NI; p.SG = SG;
    p.PH = NI > 1 ? NI * SG : 16 + pl.FH - 1; p.PW = 8 + pl.FW - 1;
    if (p.PH > 256) return 1;
    p.row_blocks = NI > 1 ? 1 : (pl.oH + 15) / 16;
    p.col_blocks = (pl.oW + 7) / 8;
    // accumulators of 4 rows x 32 patch columns where they hold more real pixels than 16 x 8 ones (option HALO_FLAT32:
    // 0 never, 2 wherever the shape allows)
    bool flat32 = false;
    if (NI == 1 && pl.oW + pl.FW - 1 <= 32 && pl.oSH == 1 && pl.oSW == 1 && pl.oNH == 0 && pl.oNW == 0 && opt(OPT_HALO_FLAT32)) {
        const long long lanes16 = (long long)p.row_blocks * p.col_blocks * 128, lanes4 = (long long)((pl.oH + 3) / 4) * 128;
        flat32 = lanes4 * 10 <= lanes16 * 9 || opt(OPT_HALO_FLAT32) == 2;
    }
    if (flat32) {
        p.PH = 4 + pl.FH - 1; p.PW = 32;
        p.row_blocks = (pl.oH + 3) / 4; p.col_blocks = 1;
    }
    p.n_blocks = (p.N + NI - 1) / NI;
    const long long per_ntile = (long long)p.n_blocks * p.row_blocks * p.col_blocks;
    if (per_ntile % 2 != 0) return 1;   // the two tiles of a pair must share their W tiles
    const long long total = per_ntile * p.n_tiles;
    if (total > 2147483647LL) return 1;
    p.total_tiles = (int)total;
    const bool wide = mode3x != 0 && !three;
    const uint32_t accw = (wide || side3) ? 2 * BN : BN;
    p.acc_bufs = 2 * accw <= 512 ? 2 : 1;
    p.mode3x = wide ? 2 : (three ? (side3 ? 4 : 1) : 0); p.b_mn = 0; p.flip = 0;
    p.idesc = make_idesc_tf32(256, BN, false, false);
    p.idesc_wide = make_idesc_tf32(256, wide ? 2 * BN : BN, false, false);
    p.tmem_cols = pow2_cols(p.acc_bufs * accw);
    p.patch_tx = (uint32_t)p.PH * p.PW * 128;
    p.patch_bytes = (p.patch_tx + 1023) & ~1023u;
    p.b_tx = wide ? (uint32_t)BN * 192 : (three ? (uint32_t)BN * 128 : (uint32_t)BN * 64);   // P + Q, hi + lo halves, or BN/2 rows
    p.b_bytes = p.b_tx;
    const uint32_t planes = mode3x ? 2 : 1;
    const size_t smem_cap = 226 * 1024;
    bool row = opt(OPT_HALO_ROW) != 0;
    p.npb = 2;
    auto need = [&](bool r, int sb) {
        return (size_t)p.npb * p.patch_bytes * planes + (size_t)sb * p.b_bytes * (r ? pl.FW : 1) + 32768 + 512 + 1024;
    };
    if (row && need(true, 2) > smem_cap) row = false;
    int sb = 2;
    if (need(row, sb) > smem_cap) return 1;
    const int max_sb = row ? pl.FH * 2 : 8;
    while (sb < max_sb && need(row, sb + 1) <= smem_cap) ++sb;
    p.sb = sb;
    const size_t smem = need(row, sb);

    CUtensorMap tmA, tmB, tmBlo, tmO;
    cuuint64_t ad[4] = {(cuuint64_t)pl.aC, (cuuint64_t)pl.aW, (cuuint64_t)pl.aH, (cuuint64_t)pl.aN};
    cuuint64_t as[3] = {(cuuint64_t)pl.aC * 4, (cuuint64_t)pl.aW * pl.aC * 4, (cuuint64_t)pl.aH * pl.aW * pl.aC * 4};
    cuuint32_t abox[4] = {32, (cuuint32_t)p.PW, (cuuint32_t)(NI > 1 ? p.SG : p.PH), (cuuint32_t)NI};
    int rc = make_tiled_map(&tmA, pl.act, 4, ad, as, abox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const float* w_hi = pl.W;
    const float* w_lo = pl.W_lo ? pl.W_lo : pl.W;
    if (mode3x && !pl.W_lo) {
        rc = forward_lo_plane(c, stream, pl.W, (size_t)pl.wOC * pl.FH * pl.FW * pl.wIC, &w_lo);
        if (rc) return rc;
    }
    cuuint64_t wd[3] = {(cuuint64_t)pl.wIC, (cuuint64_t)pl.FH * pl.FW, (cuuint64_t)pl.wOC};
    cuuint64_t wst[2] = {(cuuint64_t)pl.wIC * 4, (cuuint64_t)pl.FH * pl.FW * pl.wIC * 4};
    cuuint32_t box[3] = {32, 1, (cuuint32_t)(BN / 2)};
    rc = make_tiled_map(&tmB, w_hi, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = make_tiled_map(&tmBlo, w_lo, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const int oNH = pl.oNH ? pl.oNH : pl.oH, oNW = pl.oNW ? pl.oNW : pl.oW;
    cuuint64_t od[4] = {(cuuint64_t)pl.ncols, (cuuint64_t)pl.oW, (cuuint64_t)pl.oH, (cuuint64_t)pl.aN};
    cuuint64_t ost[3] = {(cuuint64_t)pl.oSW * pl.ncols * 4, (cuuint64_t)pl.oSH * oNW * pl.ncols * 4,
                         (cuuint64_t)oNH * oNW * pl.ncols * 4};
    cuuint32_t obox[4] = {32, (cuuint32_t)(flat32 ? 32 : 8), (cuuint32_t)(flat32 ? 4 : (NI > 1 ? pl.oH : 16)), 1};
    rc = make_tiled_map(&tmO, pl.out, 4, od, ost, obox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    int pairs = sm_budget(c) / 2;
    if (pairs > p.total_tiles / 2) pairs = p.total_tiles / 2;
    HaloLaunch L{2 * pairs, smem, stream, &tmA, &tmB, &tmBlo, &tmO, &p};
    if (flat32) { if (row) halo_pair_launch_one<3, true, true>(L); else halo_pair_launch_one<3, false, true>(L); }
    else if (row) halo_pair_launch_one<3, true>(L); else halo_pair_launch_one<3, false>(L);
    note_launch(row ? "halo_pair_row" : "halo_pair_tap");
    snprintf(g_plan, sizeof(g_plan), "halo_pair%s%s%s NI=%d BN=%d npb=%d sb=%d acc=%d", row ? "_row" : "_tap", wide ? " wide" : (three ? (side3 ? " three+side" : " three") : ""),
             flat32 ? " flat32" : "", NI, BN, p.npb, sb, p.acc_bufs);
    return check_launch("conv_halo_pair_kernel");
}

// Returns 1 when the shape is left to the per-tap kernel, 0 on launch, < 0 on error.
// ---- plain TF32, few output channels: the taps of a filter row in one MMA ----------------------------
//
// conv_tapstack_kernel: tiles of 4 output rows x CB columns (32 patch columns), all of W resident in
// shared memory, N = FW * BN columns per MMA.  The cost uses the units of plan_halo (clocks of the
// busiest CTA), so the two plans compare directly.
struct TapStackPlan {
    bool valid = false;
    int BN = 0, CB = 0, npb = 0, row_blocks = 0, col_blocks = 0;
    uint32_t patch_bytes = 0, w_tile = 0, w_bytes = 0;
    size_t smem = 0;
    double cost = 0, eff = 0;
};

static TapStackPlan plan_tapstack(const IgemmPlan& pl, int mode3x, int sm_count)
{
    TapStackPlan ts;
    const int mode = opt(OPT_HALO_TAPSTACK);
    if (!mode || mode3x || pl.b_mn || pl.sh != 1 || pl.sw != 1 || pl.kdim % 32 != 0) return ts;
    if (pl.oSH != 1 || pl.oSW != 1 || pl.oNH != 0 || pl.oNW != 0) return ts;
    if (pl.FW < 2 || pl.FW > 8 || pl.ncols % 4 != 0) return ts;
    const int BN = (pl.ncols + 15) / 16 * 16;
    if (pl.FW * BN > 256) return ts;
    const int kchunks = pl.kdim / 32;
    const int PH = 4 + pl.FH - 1;
    if (PH > 256) return ts;
    ts.BN = BN;
    ts.patch_bytes = (uint32_t)PH * 4096u;
    ts.w_tile = (uint32_t)BN * 128u;
    const size_t w_bytes = (size_t)kchunks * pl.FH * pl.FW * ts.w_tile;
    const size_t cap = 227 * 1024, fixed = 1024 + 256;   // alignment slack, barriers
    if (w_bytes > 1000000 || w_bytes + 2 * (size_t)ts.patch_bytes + fixed > cap) return ts;
    ts.w_bytes = (uint32_t)w_bytes;
    int npb = (int)((cap - fixed - w_bytes) / ts.patch_bytes);
    if (npb > 6) npb = 6;
    ts.npb = npb;
    ts.smem = w_bytes + (size_t)npb * ts.patch_bytes + fixed;
    const int max_cb = 32 - (pl.FW - 1);
    ts.col_blocks = (pl.oW + max_cb - 1) / max_cb;
    ts.CB = (pl.oW + ts.col_blocks - 1) / ts.col_blocks;
    ts.row_blocks = (pl.oH + 3) / 4;
    const long long tiles = (long long)pl.aN * ts.row_blocks * ts.col_blocks;
    if (tiles > 2147483647LL) return ts;
    ts.eff = (double)pl.oH * pl.oW / ((double)ts.row_blocks * ts.col_blocks * 128.0);
    auto clk = [](double n) { return n / 2.0 > 59.0 ? n / 2.0 : 59.0; };
    const double steps = (double)kchunks * pl.FH * 4;
    const double t_mma = steps * clk((double)pl.FW * BN) + 600.0;
    const double t_smem = (steps * (4096.0 + 32.0 * pl.FW * BN) + (double)kchunks * ts.patch_bytes + 4.0 * 128 * BN * 4) / 128.0 + 500.0;
    const double t_l2 = ((double)kchunks * ts.patch_bytes + 128.0 * BN * 4) / 28.0;
    double t = t_mma > t_smem ? t_mma : t_smem;
    if (t_l2 > t) t = t_l2;
    if (npb < 3) t *= 1.25;
    // every CTA loads all of W before its first MMA
    ts.cost = t * (double)((tiles + sm_count - 1) / sm_count) + (double)w_bytes / 28.0;
    ts.valid = mode == 2 || ts.eff >= 0.6;
    return ts;
}

static int launch_tapstack(DeviceCtx* c, const IgemmPlan& pl, const TapStackPlan& ts, cudaStream_t stream)
{
    TapStackParams p{};
    p.out = pl.out; p.bias = pl.bias; p.act_on = pl.act_on; p.act_k = pl.act_k; p.status = c->status; p.prof = c->prof;
    p.N = pl.aN; p.OH = pl.oH; p.OW = pl.oW; p.Ncols = pl.ncols; p.ldo = pl.ncols;
    p.FH = pl.FH; p.FW = pl.FW; p.pad_h = pl.pad_h; p.pad_w = pl.pad_w;
    p.kchunks = pl.kdim / 32; p.BN = ts.BN; p.CB = ts.CB;
    p.row_blocks = ts.row_blocks; p.col_blocks = ts.col_blocks;
    p.total_tiles = (int)((long long)pl.aN * ts.row_blocks * ts.col_blocks);
    p.npb = ts.npb; p.patch_bytes = ts.patch_bytes; p.w_tile = ts.w_tile; p.w_bytes = ts.w_bytes;
    p.accw = (uint32_t)pl.FW * ts.BN;
    p.idesc = make_idesc_tf32(kBM, pl.FW * ts.BN, false, false);
    // the epilogue reads 32 columns at a time; with BN % 32 != 0 its last read of a tap block runs up to 16
    // columns past the second accumulator
    p.tmem_cols = pow2_cols(2 * pl.FW * ts.BN + (ts.BN % 32 ? 32 : 0));

    CUtensorMap tmA, tmB;
    cuuint64_t ad[4] = {(cuuint64_t)pl.aC, (cuuint64_t)pl.aW, (cuuint64_t)pl.aH, (cuuint64_t)pl.aN};
    cuuint64_t as[3] = {(cuuint64_t)pl.aC * 4, (cuuint64_t)pl.aW * pl.aC * 4, (cuuint64_t)pl.aH * pl.aW * pl.aC * 4};
    cuuint32_t abox[4] = {32, 32, (cuuint32_t)(4 + pl.FH - 1), 1};
    int rc = make_tiled_map(&tmA, pl.act, 4, ad, as, abox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cuuint64_t wd[3] = {(cuuint64_t)pl.wIC, (cuuint64_t)pl.FH * pl.FW, (cuuint64_t)pl.wOC};
    cuuint64_t wst[2] = {(cuuint64_t)pl.wIC * 4, (cuuint64_t)pl.FH * pl.FW * pl.wIC * 4};
    cuuint32_t wbox[3] = {32, 1, (cuuint32_t)ts.BN};
    rc = make_tiled_map(&tmB, pl.W, 3, wd, wst, wbox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(conv_tapstack_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(conv_tapstack_kernel<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(conv_tapstack_kernel<3, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(conv_tapstack_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr_done = true;
    }
    const int grid = sm_budget(c) < p.total_tiles ? sm_budget(c) : p.total_tiles;
    if (!t_dry) {
        if (pl.FW == 3 && pl.FH == 3) conv_tapstack_kernel<3, 3><<<grid, kTapStackThreads, ts.smem, stream>>>(tmA, tmB, p);
        else if (pl.FW == 3) conv_tapstack_kernel<3, 0><<<grid, kTapStackThreads, ts.smem, stream>>>(tmA, tmB, p);
        else if (pl.FW == 2) conv_tapstack_kernel<2, 0><<<grid, kTapStackThreads, ts.smem, stream>>>(tmA, tmB, p);
        else conv_tapstack_kernel<0, 0><<<grid, kTapStackThreads, ts.smem, stream>>>(tmA, tmB, p);
    }
    note_launch("halo_tapstack");
    snprintf(g_plan, sizeof(g_plan), "tapstack BN=%d N=%d CB=%d npb=%d eff=%.2f", ts.BN, pl.FW * ts.BN, ts.CB, ts.npb, ts.eff);
    return check_launch("conv_tapstack_kernel");
}

static int launch_halo(DeviceCtx* c, const IgemmPlan& pl_in, int mode3x, cudaStream_t stream)
{
    const int tile_mode = env_tile_mode();
    if (tile_mode == 1) return 1;
    IgemmPlan pl = pl_in;
    if (pl.sh != 1 || pl.sw != 1 || pl.kdim % 32 != 0) return 1;
    // CTA pairs: the single-CTA forms are bound by shared-memory bandwidth once an MMA covers 128 or
    // more columns (operand reads alone take 128 B/clk at N = 128), and a pair halves the W-tile part
    // of it.  Measured faster in plain TF32 where one MMA covers 256 output channels (OC % 256 == 0:
    // 14x14x256 forward 0.111 -> 0.096 ms) and in 3xTF32 with blocks of 128 channels (three MMAs with
    // side columns: 28x28x128 0.304 -> 0.287 ms, 14x14x256 0.294 -> 0.281 ms); with 64-column MMAs
    // the single-CTA forms win.  ALPHA_HALO_PAIR = 0
    // never, 1 always (wide 3xTF32), 2 always (three-MMA 3xTF32, one accumulator), 3 always (three MMAs,
    // correction terms in side columns).
    const int pair_env = opt(OPT_HALO_PAIR);
    const bool pair_auto = mode3x ? pl.ncols % 128 == 0 : pl.ncols % 256 == 0;
    // few output tiles and a long reduction: the single-CTA kernel splits the reduction over the idle SMs
    bool skinny = false;
    if (opt(OPT_SKINNY) && !pl.w_img_rows && pl.oSH == 1 && pl.oSW == 1 && pl.oNH == 0 && pl.oNW == 0) {
        const int sg = pl.oH + pl.FH - 1;
        const int ni = (sg <= 16 && opt(OPT_HALO_STACK)) ? 1 + (16 - pl.oH) / sg : 1;
        const long long tiles128 = (long long)((pl.aN + ni - 1) / ni) * (ni > 1 ? 1 : (pl.oH + 15) / 16) * ((pl.oW + 7) / 8) *
                                   ((pl.ncols + 127) / 128);
        skinny = 2 * tiles128 <= sm_budget(c) && (long long)(pl.kdim / 32) * pl.FH * pl.FW >= 32;
    }
    // per-image weights: only the single-CTA kernel knows them (its W-tile loads add the image's first row)
    const bool try_pair = !pl.w_img_rows && (pair_env > 0 || (pair_env < 0 && pair_auto && tile_mode == 0));
    if (try_pair && !skinny) {
        const int rc2 = launch_halo_pair(c, pl, mode3x, stream);
        if (rc2 != 1) return rc2;
    }
    // a 1x1 convolution does not care which pixels are neighbours: seen as one image of 8 columns
    // every 16 x 8 tile is full, whatever the real image size
    const long long flat_m = (long long)pl.aN * pl.aH * pl.aW;
    if (pl.FH == 1 && pl.FW == 1 && pl.pad_h == 0 && pl.pad_w == 0 && pl.oSH == 1 && pl.oSW == 1 && pl.oNH == 0 &&
        pl.oNW == 0 && pl.oH == pl.aH && pl.oW == pl.aW && flat_m % 8 == 0 && flat_m / 8 <= 2147483647LL &&
        opt(OPT_HALO_FLAT) && !pl.w_img_rows) {
        pl.aN = 1; pl.aW = 8; pl.aH = (int)(flat_m / 8);
        pl.oH = pl.aH; pl.oW = 8;
    }
    const int gran = pl.b_mn ? 32 : 16;
    int BN = ((pl.ncols + gran - 1) / gran) * gran;
    if (BN > 256) BN = (pl.ncols % 256 == 0 || pl.ncols > 512) ? 256 : 128;
    HaloChoice ch = plan_halo(pl, BN, mode3x, pl.b_mn, sm_budget(c));
    // narrower column tiles when the wide ones leave SMs idle (small images, few pixels): the plan's
    // cost is the time of the busiest CTA, so candidates compare directly
    for (int cand = 128; cand >= 64; cand >>= 1) {
        if (cand >= BN || pl.ncols % cand != 0 || !opt(OPT_HALO_NARROW)) continue;
        HaloChoice alt = plan_halo(pl, cand, mode3x, pl.b_mn, sm_budget(c));
        if (alt.valid && (!ch.valid || alt.cost < 0.9 * ch.cost)) { ch = alt; BN = cand; }
    }
    {
        // plain TF32 with few output channels: one MMA per filter row where the model says it is faster
        const TapStackPlan ts = pl.w_img_rows ? TapStackPlan{} : plan_tapstack(pl, mode3x, sm_budget(c));
        if (ts.valid && (opt(OPT_HALO_TAPSTACK) == 2 || !ch.valid || ts.cost < 0.8 * ch.cost)) return launch_tapstack(c, pl, ts, stream);
    }
    if (!ch.valid || (tile_mode == 0 && ch.eff < 0.6 && !pl.force)) {
        // a skinny shape whose tiles the single-CTA kernel would leave mostly empty: the pair kernel after all
        if (try_pair && skinny) {
            const int rc2 = launch_halo_pair(c, pl_in, mode3x, stream);
            if (rc2 != 1) return rc2;
        }
        return 1;
    }

    HaloParams p{};
    p.out = pl.out; p.bias = pl.bias; p.act_on = pl.act_on; p.act_k = pl.act_k; p.status = c->status; p.prof = c->prof;
    p.N = pl.aN; p.OH = pl.oH; p.OW = pl.oW;
    p.Ncols = pl.ncols; p.ldo = pl.ncols;
    p.FH = pl.FH; p.FW = pl.FW; p.pad_h = pl.pad_h; p.pad_w = pl.pad_w;
    p.kchunks = pl.kdim / 32;
    p.BN = BN; p.n_tiles = (pl.ncols + BN - 1) / BN;
    p.JH = ch.JH; p.JW = ch.JW;
    p.NI = ch.NI; p.SG = pl.oH + pl.FH - 1;
    p.PH = ch.NI > 1 ? ch.NI * p.SG : 16 * ch.JH + pl.FH - 1; p.PW = 8 * ch.JW + pl.FW - 1;
    p.row_blocks = ch.NI > 1 ? 1 : (pl.oH + 16 * ch.JH - 1) / (16 * ch.JH);
    p.col_blocks = (pl.oW + 8 * ch.JW - 1) / (8 * ch.JW);
    p.n_blocks = (p.N + ch.NI - 1) / ch.NI;
    const int Jflat = ch.JH * ch.JW;
    if (ch.flat) {
        // the macro tiles index the list of all four-row blocks of the batch: row_blocks of them, in one "image block"
        p.flat = 1; p.flat_rb4 = (pl.oH + 3) / 4;
        const long long blocks = (long long)p.N * p.flat_rb4;
        if (blocks > 2147483647LL) return 1;
        p.flat_total = (int)blocks;
        p.PH = 4 + pl.FH - 1; p.PW = 32;
        p.n_blocks = 1; p.col_blocks = 1; p.row_blocks = (int)((blocks + Jflat - 1) / Jflat);
    }
    const long long total = (long long)p.n_tiles * p.n_blocks * p.row_blocks * p.col_blocks;
    if (total > 2147483647LL) return 1;
    p.total_tiles = (int)total;
    p.npb = ch.npb; p.sb = ch.sb; p.acc_bufs = ch.acc_bufs;
    p.mode3x = ch.wide ? 2 : mode3x; p.b_mn = pl.b_mn; p.flip = pl.flip;
    p.w_img_rows = pl.w_img_rows;
    // plain TF32 is bound by one thread's MMA issue interval, not by the tensor pipe: two issuing
    // threads alternate over the ring's stages (the ring then needs an even number of slots).
    // The 3xTF32 forms run N >= 128 per MMA, are pipe-bound and keep one issuer (and with it a
    // fixed accumulation order).
    p.dual = (p.mode3x == 0 && p.sb >= 2 && opt(OPT_HALO_DUAL)) ? 1 : 0;
    if (p.dual) p.sb &= ~1;
    p.idesc = make_idesc_tf32(kBM, BN, false, pl.b_mn);
    p.idesc_wide = make_idesc_tf32(kBM, ch.wide ? 2 * BN : BN, false, pl.b_mn);
    p.tmem_cols = pow2_cols(ch.acc_bufs * ch.JH * ch.JW * BN * (ch.wide ? 2 : 1));
    p.patch_tx = (uint32_t)p.PH * p.PW * 128 * (ch.flat ? Jflat : 1);
    p.patch_bytes = (p.patch_tx + 1023) & ~1023u;
    p.b_tx = pl.b_mn ? (BN / 32) * 4096 : BN * 128;
    p.b_bytes = (p.b_tx + 1023) & ~1023u;
    const uint32_t planes = mode3x ? 2 : 1;
    const int tps = ch.row ? pl.FW : 1;
    const size_t smem = (size_t)p.npb * p.patch_bytes * planes + (size_t)p.sb * p.b_bytes * planes * tps + 32768 +
                        (3 * p.npb + 3 * p.sb + 8) * 8 + 1024;

    CUtensorMap tmA, tmB;
    cuuint64_t ad[4] = {(cuuint64_t)pl.aC, (cuuint64_t)pl.aW, (cuuint64_t)pl.aH, (cuuint64_t)pl.aN};
    cuuint64_t as[3] = {(cuuint64_t)pl.aC * 4, (cuuint64_t)pl.aW * pl.aC * 4, (cuuint64_t)pl.aH * pl.aW * pl.aC * 4};
    cuuint32_t abox[4] = {32, (cuuint32_t)p.PW, (cuuint32_t)(ch.NI > 1 ? p.SG : p.PH), (cuuint32_t)ch.NI};
    int rc = make_tiled_map(&tmA, pl.act, 4, ad, as, abox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    // 3xTF32: split W into hi/lo planes once per call (scratch of this stream), load both by TMA
    const float* w_hi = pl.W;
    const float* w_lo = pl.W_lo ? pl.W_lo : pl.W;
    // Option HALO_SPLITB (off by default): a 1x1 product loads only W itself and its split warps form the lo
    // plane of each W tile in shared memory, which halves the W traffic out of L2 and drops the pass over W.
    // Measured: no gain on the L2-bound tiny-image layers (3.84 against 3.82 ms for the ResNet-18 stack) and a
    // loss on large products (8192^3 C = A * B^T: 187 against 212 TFLOP/s), where the extra shared-memory
    // traffic of the split competes with the operand reads of the MMAs.
    p.split_b = (mode3x && !pl.W_lo && !pl.b_mn && pl.FH * pl.FW == 1 && opt(OPT_HALO_SPLITB) &&
                 !(t_prepared_lo.W == pl.W && t_prepared_lo.lo)) ? 1 : 0;
    if (mode3x && !pl.W_lo && !p.split_b) {
        rc = forward_lo_plane(c, stream, pl.W, (size_t)pl.wOC * pl.FH * pl.FW * pl.wIC, &w_lo);
        if (rc) return rc;
    }
    CUtensorMap tmBlo, tmO;
    cuuint64_t wd[3] = {(cuuint64_t)pl.wIC, (cuuint64_t)pl.FH * pl.FW, (cuuint64_t)pl.wOC};
    cuuint64_t wst[2] = {(cuuint64_t)pl.wIC * 4, (cuuint64_t)pl.FH * pl.FW * pl.wIC * 4};
    if (!pl.b_mn) {
        cuuint32_t box[3] = {32, 1, (cuuint32_t)BN};
        rc = make_tiled_map(&tmB, w_hi, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (!rc) rc = make_tiled_map(&tmBlo, w_lo, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        cuuint32_t box[3] = {32, 1, 32};
        rc = make_tiled_map(&tmB, w_hi, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        if (!rc) rc = make_tiled_map(&tmBlo, w_lo, 3, wd, wst, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    }
    if (rc) return rc;
    // Split-K: a layer with few output tiles and a long reduction (small images or batch, many channels)
    // would leave most SMs idle while a handful of CTAs stream the whole filter.  Every tile is then
    // computed as ksplit partial sums over disjoint ranges of the reduction chunks, each by its own
    // CTA, into scratch laid out as ksplit copies of the output; a second kernel adds them in order
    // (with the bias and the activation, which the partial sums must not see).
    const int ksplit = ch.flat ? 1 : halo_ksplit(pl, p.total_tiles, p.kchunks, sm_budget(c));
    p.cps = (p.kchunks + ksplit - 1) / ksplit;
    p.ksplit = ksplit;
    float* out_ptr = pl.out;
    const size_t out_floats = (size_t)pl.aN * pl.oH * pl.oW * pl.ncols;
    if (ksplit > 1) {
        if ((long long)pl.aN * ksplit > 2147483647LL) return 1;
        rc = get_workspace(c, stream, (size_t)ksplit * out_floats * sizeof(float), &out_ptr);
        if (rc) return rc;
        p.bias = nullptr; p.act_on = 0;
    }
    // output [N][OH][OW][ldo] for the epilogue's TMA stores: one slab = 32 channels x 8 columns x 16 rows
    const int oNH = pl.oNH ? pl.oNH : pl.oH, oNW = pl.oNW ? pl.oNW : pl.oW;
    cuuint64_t od[4] = {(cuuint64_t)pl.ncols, (cuuint64_t)pl.oW, (cuuint64_t)pl.oH, (cuuint64_t)pl.aN * ksplit};
    cuuint64_t ost[3] = {(cuuint64_t)pl.oSW * pl.ncols * 4, (cuuint64_t)pl.oSH * oNW * pl.ncols * 4,
                         (cuuint64_t)oNH * oNW * pl.ncols * 4};
    cuuint32_t obox[4] = {32, (cuuint32_t)(ch.flat ? 32 : 8), (cuuint32_t)(ch.flat ? 4 : (ch.NI > 1 ? pl.oH : 16)), 1};
    rc = make_tiled_map(&tmO, out_ptr, 4, od, ost, obox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const long long vtiles = (long long)p.total_tiles * ksplit;
    int grid = sm_budget(c) < vtiles ? sm_budget(c) : (int)vtiles;
    HaloLaunch L{grid, smem, stream, &tmA, &tmB, &tmBlo, &tmO, &p};
    if (ch.flat) { if (ch.row) halo_launch_one<3, 2, 1, true, true>(L); else halo_launch_one<3, 2, 1, false, true>(L); }
    else if (!ch.stat) halo_launch_one<0, 0, 0, false>(L);
    else if (pl.FW == 1) halo_launch_fw<1>(L, ch.JH, ch.JW, ch.row);
    else if (pl.FW == 2) halo_launch_fw<2>(L, ch.JH, ch.JW, ch.row);
    else if (pl.FW == 3) halo_launch_fw<3>(L, ch.JH, ch.JW, ch.row);
    else halo_launch_fw<5>(L, ch.JH, ch.JW, ch.row);
    note_launch(ch.row ? "halo_row" : (ch.stat ? "halo_tap" : "halo"));
    snprintf(g_plan, sizeof(g_plan), "halo%s%s%s%s JH=%d JW=%d NI=%d BN=%d npb=%d sb=%d acc=%d eff=%.2f ksplit=%d", ch.row ? "_row" : (ch.stat ? "_tap" : ""),
             ch.wide ? " wide" : "", p.dual ? " dual" : "", ch.flat ? " flat32" : "", ch.JH, ch.JW, ch.NI, BN, ch.npb, p.sb, ch.acc_bufs, ch.eff, ksplit);
    rc = check_launch("conv_halo_kernel");
    if (rc || ksplit == 1) return rc;
    const size_t n4 = out_floats / 4;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > (size_t)c->sm_count * 8) blocks = (size_t)c->sm_count * 8;
    if (!t_dry) splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(out_ptr), n4, ksplit, pl.bias, pl.ncols / 4,
                                                               pl.act_on, pl.act_k, reinterpret_cast<float4*>(pl.out));
    note_launch(ch.row ? "halo_row" : (ch.stat ? "halo_tap" : "halo"));
    return check_launch("splitk_reduce_kernel");
}

// ---- channel counts the tensor kernels cannot stage: patch matrix + 1x1 convolution ---------------
//
// The forward kernels stage 8, 16 or 32 input channels per filter tap and the deltaW kernels 32,
// so a first layer with IC = 4 (3 colour planes padded to 4) would fall to the gather kernels.
// Instead the patches are written out once as a matrix A[N*OH*OW][Kp], Kp = FH*FW*IC rounded up to
// 32 with zero columns, and the convolution becomes a 1x1 convolution over an "image" with Kp
// channels: forward Y = A * W^T with W read in place as [OC][FH*FW*IC] (the tensor map zero-fills
// the columns past FH*FW*IC), deltaW = deltaY^T * A, unpadded afterwards.
static int make_patch_matrix(DeviceCtx* c, PatchShape ps, const float* X, cudaStream_t stream, float** A, int* K_out,
                             int* Kp_out, size_t extra_floats)
{
    const int K = ps.FH * ps.FW * ps.IC, Kp = (K + 31) / 32 * 32;
    ps.K = K; ps.Kp = Kp;
    const size_t M = (size_t)ps.N * ps.OH * ps.OW;
    float* ws = nullptr;
    int rc = get_workspace(c, stream, (M * Kp + extra_floats) * sizeof(float), &ws, 1);
    if (rc) return rc;
    const size_t total = M * (Kp / 4);
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
    const bool idx32 = M * (size_t)Kp <= 2147483647ull && (size_t)ps.N * ps.IH * ps.IW * ps.IC <= 2147483647ull;
    if (idx32) {
        const PatchDivs dv{fast_div(Kp / 4), fast_div(ps.IC), fast_div(ps.FW), fast_div(ps.OW), fast_div(ps.OH)};
        if (!t_dry) patch_matrix32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(X, ws, ps, dv);
    } else {
        if (!t_dry) patch_matrix_kernel<<<(unsigned)blocks, 256, 0, stream>>>(X, ws, ps);
    }
    note_launch("patch_matrix");
    rc = check_launch("patch_matrix_kernel");
    if (rc) return rc;
    *A = ws; *K_out = K; *Kp_out = Kp;
    return ALPHA_OK;
}

static PatchShape patch_shape_of(const AlphaConvShape* s)
{
    return PatchShape{s->N, s->IH, s->IW, s->IC, s->FH, s->FW, s->OH, s->OW, s->sh, s->sw, s->ph, s->pw, 0, 0};
}

// Forward-form plan (K-major weights [wOC][taps][wIC], any stride) as patch matrix + 1x1 convolution.
// Returns 1 when no tensor kernel takes the 1x1 problem.
static int launch_patch_gemm(DeviceCtx* c, const IgemmPlan& pl, int mode3x, cudaStream_t stream)
{
    PatchShape ps{pl.aN, pl.aH, pl.aW, pl.aC, pl.FH, pl.FW, pl.oH, pl.oW, pl.sh, pl.sw, pl.pad_h, pl.pad_w, 0, 0};
    float* A = nullptr;
    int K = 0, Kp = 0;
    int rc = make_patch_matrix(c, ps, pl.act, stream, &A, &K, &Kp, 0);
    if (rc) return rc;
    IgemmPlan g = pl;
    g.act = A; g.aH = pl.oH; g.aW = pl.oW; g.aC = Kp;
    g.FH = 1; g.FW = 1; g.sh = 1; g.sw = 1; g.pad_h = 0; g.pad_w = 0;
    g.wIC = K; g.kdim = Kp; g.b_mn = false; g.flip = false; g.force = true;
    rc = launch_halo(c, g, mode3x, stream);
    if (rc != 1) return rc;
    if (g.W_lo) return 1;   // the per-tap kernel splits W itself and cannot take pre-split planes
    return launch_igemm(c, g, mode3x, stream);
}

// Images so small that the 16 x 8 pixel tiles of the halo kernel stay mostly empty
static bool tiny_image(int oH, int oW) { return oH * oW <= 16; }

static bool patch_path_ok(const AlphaConvShape* s)
{
    const long long K = (long long)s->FH * s->FW * s->IC;
    return s->IC % 4 == 0 && K <= 16384 && opt(OPT_PATCH_MATRIX) != 0;
}

static bool taps_fit64(const AlphaConvShape* s) { return s->FH * s->FW <= 64; }

// ---- strided deltaX: one stride-1 convolution per output phase ------------------------------------
//
// deltaX[n, sh*a + py, sw*b + px, :] only receives the filter taps fh = ry + sh*u, fw = rx + sw*v with
// ry = (py + ph) % sh, rx = (px + pw) % sw.  Each of the sh*sw phases is therefore a stride-1
// convolution of deltaY with a sub-filter (the reference's "kernel split",
// Cuda_dconv3D_deltaX/dconv3D_dX_kernelSplit_remode_v2.cuh:35-66), run on the halo kernel with the
// phase's weights transposed and pre-split, and written through a tensor map that addresses every
// sh-th row and sw-th column of deltaX.
// Returns 1 when the shape is left to the gather kernel, 0 when all phases were launched, < 0 on error.
static int launch_dx_phases(DeviceCtx* c, const AlphaConvShape* s, const float* dY, const float* W, float* dX,
                            int mode3x, cudaStream_t stream)
{
    if (env_tile_mode() == 1 || !opt(OPT_DX_PHASES)) return 1;
    if (s->OC % 32 != 0 || s->sh > 8 || s->sw > 8 || !taps_fit64(s)) return 1;
    if (s->IH < s->sh || s->IW < s->sw) return 1;
    if (s->FH < s->sh || s->FW < s->sw) {
        // some phases receive no filter tap at all (1x1 stride 2): those pixels of deltaX are zero
        cudaError_t e = t_dry ? cudaSuccess : cudaMemsetAsync(dX, 0, (size_t)s->N * s->IH * s->IW * s->IC * sizeof(float), stream);
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemsetAsync(deltaX): %s", cudaGetErrorString(e));
    }
    const int taps = s->FH * s->FW;
    const size_t nW = (size_t)s->OC * taps * s->IC;
    float* ws = nullptr;
    bool fresh = true;
    const DeviceCtx::WeightKey wkey{W, WK_DX_PHASES, s->OC, s->IC, s->FH * 256 + s->FW,
                                    (s->sh << 24) | (s->sw << 16) | (s->ph << 8) | s->pw, mode3x};
    int rc = weight_planes(c, stream, wkey, (mode3x ? 2 : 1) * nW * sizeof(float), &ws, &fresh);
    if (rc) return rc;
    size_t woff = 0;
    for (int py = 0; py < s->sh; ++py)
        for (int px = 0; px < s->sw; ++px) {
            const int ry = (py + s->ph) % s->sh, rx = (px + s->pw) % s->sw;
            const int Uy = (s->FH - ry + s->sh - 1) / s->sh, Ux = (s->FW - rx + s->sw - 1) / s->sw;
            const int qy = (py + s->ph - ry) / s->sh, qx = (px + s->pw - rx) / s->sw;
            const int A = (s->IH - py + s->sh - 1) / s->sh, Bw = (s->IW - px + s->sw - 1) / s->sw;
            const int ptaps = Uy * Ux;
            if (ptaps == 0) continue;
            TapMap map{};
            map.n = ptaps;
            for (int u = 0; u < Uy; ++u)
                for (int v = 0; v < Ux; ++v)
                    map.src[u * Ux + v] = (ry + s->sh * (Uy - 1 - u)) * s->FW + (rx + s->sw * (Ux - 1 - v));
            const size_t pn = (size_t)s->OC * ptaps * s->IC;
            float* whi = ws + woff;
            float* wlo = mode3x ? ws + nW + woff : nullptr;
            woff += pn;
            if (fresh) {
                dim3 tg((s->IC + 31) / 32, (s->OC + 31) / 32, ptaps);
                if (transforms_run()) transpose_weights_kernel<<<tg, 256, 0, stream>>>(W, whi, wlo, s->OC, s->IC, taps, map, mode3x);
                note_launch("transpose_w");
                rc = check_launch("transpose_weights_kernel");
                if (rc) return rc;
            }
            IgemmPlan pl{};
            pl.act = dY; pl.aN = s->N; pl.aH = s->OH; pl.aW = s->OW; pl.aC = s->OC;
            pl.FH = Uy; pl.FW = Ux; pl.sh = 1; pl.sw = 1;
            pl.pad_h = Uy - 1 - qy; pl.pad_w = Ux - 1 - qx;
            pl.out = dX + ((size_t)py * s->IW + px) * s->IC;
            pl.oH = A; pl.oW = Bw; pl.ncols = s->IC;
            pl.oSH = s->sh; pl.oSW = s->sw; pl.oNH = s->IH; pl.oNW = s->IW;
            pl.W = whi; pl.W_lo = wlo; pl.wOC = s->IC; pl.wIC = s->OC; pl.bias = nullptr;
            pl.b_mn = false; pl.flip = false; pl.kdim = s->OC; pl.force = true;
            if (tiny_image(A, Bw) && (long long)ptaps * s->OC <= 16384 && ptaps * s->OC >= 2048 &&
                opt(OPT_PATCH_MATRIX)) {
                // phases of a few pixels per image: patch matrix of deltaY, dense 1x1 product, scatter
                PatchShape ps{s->N, s->OH, s->OW, s->OC, Uy, Ux, A, Bw, 1, 1, pl.pad_h, pl.pad_w, 0, 0};
                const size_t M = (size_t)s->N * A * Bw;
                float* P = nullptr;
                int K = 0, Kp = 0;
                const WsMark mark = ws_mark(c, stream);   // every phase reuses the same patch-matrix bytes
                rc = make_patch_matrix(c, ps, dY, stream, &P, &K, &Kp, M * s->IC);
                if (rc) return rc;
                float* Sp = P + M * Kp;
                IgemmPlan g = pl;
                g.act = P; g.aH = A; g.aW = Bw; g.aC = Kp; g.FH = 1; g.FW = 1; g.pad_h = 0; g.pad_w = 0;
                g.out = Sp; g.oSH = 1; g.oSW = 1; g.oNH = 0; g.oNW = 0;
                g.wIC = K; g.kdim = Kp;
                rc = launch_halo(c, g, mode3x, stream);
                if (rc == 1) return fail(ALPHA_E_ARG, "strided deltaX: phase (%d,%d) does not fit the halo kernel", py, px);
                if (rc) return rc;
                const size_t total4 = M * (s->IC / 4);
                size_t blocks = (total4 + 255) / 256;
                if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
                if (!t_dry) scatter_phase_kernel<<<(unsigned)blocks, 256, 0, stream>>>(Sp, pl.out, s->N, A, Bw, s->IC, s->sh, s->sw, s->IH, s->IW);
                note_launch("dx_patch");
                rc = check_launch("scatter_phase_kernel");
                if (rc) return rc;
                ws_rewind(c, stream, mark);
                continue;
            }
            rc = launch_halo(c, pl, mode3x, stream);
            if (rc == 1) return fail(ALPHA_E_ARG, "strided deltaX: phase (%d,%d) does not fit the halo kernel", py, px);
            if (rc) return rc;
        }
    if (fresh) weight_planes_ready(c, stream, wkey);
    return ALPHA_OK;
}

// ---- deltaX with few input channels (image planes): 1x1 product + col2im ---------------------------
//
// With IC = 4 the phase kernels would run MMAs of 16 columns.  Instead P = deltaY x Wt as a 1x1
// convolution with IC * FH * FW output columns (Wt[ic][tap][oc], what transpose_weights_kernel
// writes), then every input pixel gathers its taps from P.  Any stride.
// Returns 1 when the shape is left to the other paths.
static int launch_dx_col2im(DeviceCtx* c, const AlphaConvShape* s, const float* dY, const float* W, float* dX, int mode3x,
                            cudaStream_t stream)
{
    const int taps = s->FH * s->FW;
    const long long cols = (long long)s->IC * taps;
    if (s->IC % 4 != 0 || s->OC % 32 != 0 || taps > 64) return 1;
    if (!opt(OPT_DX_COL2IM) || env_tile_mode() == 1) return 1;
    const size_t M = (size_t)s->N * s->OH * s->OW, nW = (size_t)s->OC * cols;
    // Image planes (IC <= 8): always.  More channels: while the product matrix P[pixels][taps * IC] stays
    // small enough to live in the L2 cache between the kernel that writes it and the one that gathers
    // from it, one dense product beats sh * sw phase convolutions with a few taps each; larger P would
    // cost 2 * |P| of HBM traffic and the phases win.
    const bool planes = s->IC <= 8 && cols <= 512;
    const bool small_p = opt(OPT_DX_COL2IM) >= 1 && M * (size_t)cols * sizeof(float) <= (size_t)96 << 20 && cols <= 65536;
    // Phase images of a few pixels (a 4x4 s2 generator layer growing 4x4 to 8x8: four phases of 4x4 pixels) fill a
    // fraction of a 16 x 8 pixel accumulator tile, while the dense product has no idle lane and no wasted product
    // (every deltaY pixel times every tap is used exactly once), so it wins although P then passes through HBM:
    // phases of at most 4x4 pixels in both math modes, of at most 8x8 in 3xTF32, whose longer MMAs hide the passes
    // over P (batch 1024, 4x4 s2: 8x8x256 from 4x4x512 0.72 -> 0.41 ms, 16x16x128 from 8x8x256 0.88 -> 0.53 ms).
    const int pa = (s->IH + s->sh - 1) / s->sh, pb = (s->IW + s->sw - 1) / s->sw;
    const bool tiny_phase = (s->sh > 1 || s->sw > 1) && opt(OPT_DX_COL2IM) >= 1 && cols <= 65536 && s->IC % 32 == 0 &&
                            M * (size_t)cols * sizeof(float) <= (size_t)2 << 30 && (pa * pb <= 16 || (mode3x && pa * pb <= 64));
    const bool forced_p = opt(OPT_DX_COL2IM) == 2 && cols <= 65536 && M * (size_t)cols * sizeof(float) <= (size_t)8 << 30;
    if (!planes && !small_p && !tiny_phase && !forced_p) return 1;
    const int tap_major = planes ? 0 : 1;
    float* ws = nullptr;
    bool fresh = true;
    const DeviceCtx::WeightKey wkey{W, WK_DX_COL2IM, s->OC, s->IC, s->FH * 256 + s->FW, tap_major, mode3x};
    int rc = weight_planes(c, stream, wkey, (mode3x ? 2 : 1) * nW * sizeof(float), &ws, &fresh);
    if (rc) return rc;
    float* P = nullptr;
    rc = get_workspace(c, stream, M * cols * sizeof(float), &P, 1);
    if (rc) return rc;
    if (fresh) {
        TapMap map{};
        map.n = taps;
        for (int t = 0; t < taps; ++t) map.src[t] = t;
        dim3 tg((s->IC + 31) / 32, (s->OC + 31) / 32, taps);
        if (transforms_run()) transpose_weights_kernel<<<tg, 256, 0, stream>>>(W, ws, mode3x ? ws + nW : nullptr, s->OC, s->IC, taps, map, mode3x, tap_major);
        note_launch("transpose_w");
        rc = check_launch("transpose_weights_kernel");
        if (rc) return rc;
        weight_planes_ready(c, stream, wkey);
    }
    IgemmPlan pl{};
    pl.act = dY; pl.aN = s->N; pl.aH = s->OH; pl.aW = s->OW; pl.aC = s->OC;
    pl.FH = 1; pl.FW = 1; pl.sh = 1; pl.sw = 1; pl.pad_h = 0; pl.pad_w = 0;
    pl.out = P; pl.oH = s->OH; pl.oW = s->OW; pl.ncols = (int)cols;
    pl.W = ws; pl.W_lo = mode3x ? ws + nW : nullptr; pl.wOC = (int)cols; pl.wIC = s->OC; pl.bias = nullptr;
    pl.b_mn = false; pl.flip = false; pl.kdim = s->OC; pl.force = true;
    rc = launch_halo(c, pl, mode3x, stream);
    if (rc == 1) return 1;
    if (rc) return rc;
    PatchShape ps{s->N, s->IH, s->IW, s->IC, s->FH, s->FW, s->OH, s->OW, s->sh, s->sw, s->ph, s->pw, 0, 0};
    const size_t total = (size_t)s->N * s->IH * s->IW * (s->IC / 4);
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
    const bool idx32 = total * 4 <= 2147483647ull && M * (size_t)cols <= 2147483647ull;   // dX and P indexable in 31 bits
    if (idx32) {
        const GatherDivs dv{fast_div(s->IC / 4), fast_div(s->IW), fast_div(s->IH), fast_div(s->sh), fast_div(s->sw)};
        if (!t_dry) {
            if (tap_major) col2im_gather_tapmajor32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(P, dX, ps, dv);
            else col2im_gather32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(P, dX, ps, dv);
        }
    } else if (tap_major) {
        if (!t_dry) col2im_gather_tapmajor_kernel<<<(unsigned)blocks, 256, 0, stream>>>(P, dX, ps);
    } else {
        if (!t_dry) col2im_gather_kernel<<<(unsigned)blocks, 256, 0, stream>>>(P, dX, ps);
    }
    note_launch("dx_col2im");
    return check_launch("col2im_gather_kernel");
}

// ---- deltaW, halo-tile kernel (strides 1 and 2): plan and launch -----------------------------------

template <int FW_T, int R_T, int CW_T, bool STR_T = false>
static void dw_halo_set_attr()
{
    cudaFuncSetAttribute(conv_dw_halo_kernel<FW_T, R_T, CW_T, STR_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}
static inline int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

// Returns 1 when the shape is left to the split-K im2col kernel, 0 on launch, < 0 on error.
// deltaB != nullptr: the kernel also sums the columns of deltaY (bias gradient); *bias_fused tells whether it did.
// per_image: dW receives N separate results, dW[n] = the sum over the pixels of image n only (batched matrix
// products C[n] = A[n]^T * B[n]); every CTA column of the grid then owns one image and writes its result in place.
static int launch_dw_halo(DeviceCtx* c, const AlphaConvShape* s_in, const float* X, const float* dY, float* dW,
                          int mode3x, cudaStream_t stream, float* deltaB = nullptr, bool* bias_fused = nullptr,
                          bool per_image = false)
{
    if (bias_fused) *bias_fused = false;
    if (opt(OPT_CONV_DW) == 1 && !per_image) return 1;
    AlphaConvShape flat = *s_in;
    const AlphaConvShape* s = s_in;
    // a 1x1 deltaW sums over pixels in any order: one image of 16 columns fills every pixel tile
    const long long flat_m = (long long)s_in->N * s_in->OH * s_in->OW;
    if (s_in->FH == 1 && s_in->FW == 1 && s_in->ph == 0 && s_in->pw == 0 && s_in->sh == 1 && s_in->sw == 1 &&
        s_in->IH == s_in->OH && s_in->IW == s_in->OW && flat_m % 16 == 0 && flat_m / 16 <= 2147483647LL &&
        opt(OPT_HALO_FLAT) && !per_image) {
        flat.N = 1; flat.OW = flat.IW = 16; flat.OH = flat.IH = (int)(flat_m / 16);
        s = &flat;
    }
    if (s->sh < 1 || s->sh > 2 || s->sw < 1 || s->sw > 2 || s->IC % 32 != 0) return 1;
    const bool strided = s->sh != 1 || s->sw != 1;
    if (strided && (per_image || !opt(OPT_DW_STRIDED))) return 1;
    if (s->FW > 8 || s->ph >= s->FH || s->pw >= s->FW) return 1;
    // column phases of the taps: tap fw meets lattice column floor((fw - pw) / sw) + (output column) of phase (fw - pw) mod sw
    int nph = 0, ph_psi[2] = {0, 0}, ph_qmin[2] = {0, 0}, ph_qmax[2] = {0, 0}, tap_k[8], tap_q[8];
    for (int fw = 0; fw < s->FW; ++fw) {
        const int q = floor_div(fw - s->pw, s->sw), psi = fw - s->pw - q * s->sw;
        int k = 0;
        while (k < nph && ph_psi[k] != psi) ++k;
        if (k == nph) { ph_psi[k] = psi; ph_qmin[k] = ph_qmax[k] = q; ++nph; }
        if (q < ph_qmin[k]) ph_qmin[k] = q;
        if (q > ph_qmax[k]) ph_qmax[k] = q;
        tap_k[fw] = k; tap_q[fw] = q;
    }
    for (int k = 0; k < nph; ++k)
        if (ph_psi[k] >= s->IW) return 1;                 // a lattice without a column
    if (s->sh > s->IH) return 1;
    // Input channels per CTA: the accumulators of a CTA's G taps, NT columns each, must fit the 512 tensor-memory
    // columns.  A CTA owns a whole filter row (G = FW) unless rows of more than three taps do better split over
    // several CTAs of three taps (5x5, 7x7: three accumulators of 128 columns instead of five or seven of 64; an MMA of
    // N columns costs max(N / 2, 59) clocks whatever its height, and a last group with fewer taps idles its spare slots).
    struct DwForm { int G, NT; bool stacked, diag; long long cost; };
    auto mma_clk = [](int n) { return n / 2 > 59 ? n / 2 : 59; };
    auto nt_for = [&](int slots_cols, int top) {
        for (int cand = top; cand >= 32; cand >>= 1)
            if (s->IC % cand == 0 && slots_cols * cand <= 512) return cand;
        return 0;
    };
    auto pick = [&](int G) {
        DwForm f{G, nt_for(G, 256), false, false, 0};
        if (!f.NT) { f.cost = -1; return f; }
        const long long slots = (long long)((s->FW + G - 1) / G) * G;   // MMAs per 8 pixels and channel tile
        f.cost = slots * (mode3x ? 3 : 1) * mma_clk(f.NT) * ((s->OC + 127) / 128) * (s->IC / f.NT);
        // 3xTF32: three MMAs of (128 x NT), or one MMA on stacked hi/lo planes (64 + 64) x (NTq + NTq): the
        // stacked form wins where 128 output channels or 64 input channels would be half empty
        if (mode3x && !per_image) {   // the stacked form leaves two partial planes to add
            const int NTq = nt_for(2 * G, 128);
            if (NTq) {
                const long long stk_cost = slots * mma_clk(2 * NTq) * ((s->OC + 63) / 64) * (s->IC / NTq);
                bool stacked = stk_cost < f.cost;
                const int force = opt(OPT_DW_STACKED);
                if (force >= 0) stacked = force != 0;
                if (stacked) { f.stacked = true; f.NT = NTq; f.cost = stk_cost; }
            }
        }
        // plain TF32 with at most 64 output channels: two half tiles side by side ("diagonal" form), half an MMA of
        // 2 * NTd columns per 8 pixels
        if (!mode3x && !per_image && s->OC <= 64 && s->OH >= 2 && opt(OPT_DW_DIAG)) {
            const int NTd = nt_for(2 * G, 128);
            if (NTd) {
                const long long dg2 = slots * mma_clk(2 * NTd) * (s->IC / NTd);
                if (dg2 < 2 * f.cost) { f.diag = true; f.stacked = true; f.NT = NTd; f.cost = (dg2 + 1) / 2; }
            }
        }
        return f;
    };
    DwForm form = pick(s->FW);
    if (s->FW > 3 && !strided && !per_image && opt(OPT_DW_TAPGROUPS)) {
        // groups of three run the kernel whose MMAs are straight-line code; a whole row of four or more taps runs the
        // looped form, whose issuing thread needs about twice as long per MMA (5x5, 64 -> 128 channels at 112 x 112
        // in plain TF32: 3.06 ms as one row of five, 1.50 ms as 3 + 2 although that issues six MMAs for five taps)
        const DwForm g3 = pick(3);
        if (g3.cost >= 0 && (form.cost < 0 || 10 * g3.cost <= 16 * form.cost || opt(OPT_DW_TAPGROUPS) == 2)) form = g3;
    }
    if (form.cost < 0) return 1;
    const int G = form.G, tgroups = (s->FW + G - 1) / G;
    int NT = form.NT;
    const bool stacked = form.stacked, diag = form.diag;
    const int oc_tile = stacked ? 64 : 128, dyb = stacked ? 2 : 4, nsub = stacked ? 2 : 1;
    DwHaloParams p{};
    p.status = c->status; p.prof = c->prof;
    p.N = s->N; p.OH = s->OH; p.OW = s->OW;
    p.IC = s->IC; p.OC = s->OC; p.FH = s->FH; p.FW = s->FW; p.ph = s->ph; p.pw = s->pw;
    p.NT = NT; p.ic_tiles = s->IC / NT; p.oc_tiles = (s->OC + oc_tile - 1) / oc_tile;
    const int groups = tgroups * s->FH * p.ic_tiles * p.oc_tiles;
    if (groups > 65535) return 1;
    p.G = G; p.tgroups = tgroups;
    // pixel tile: CW columns of 8-pixel groups, R rows, sized so that three stages fit shared memory
    const int planes = (mode3x || diag) ? 2 : 1;   // diagonal: the second plane holds the second half tile
    int CW = opt(OPT_DW_CW);
    if (!CW) CW = (s->OW <= 8 || (s->OW % 16 != 0 && s->OW % 16 <= 8)) ? 8 : 16;  // fewer idle columns
    const int PW = CW + G - 1;
    int R = opt(OPT_DW_R);
    auto stage_bytes = [&](int r) {
        const uint32_t dyblk = ((uint32_t)r * CW * 128 + 1023) & ~1023u, xbk = ((uint32_t)r * PW * 128 + 1023) & ~1023u;
        return (size_t)planes * (dyb * dyblk + (size_t)nph * (NT / 32) * xbk);
    };
    if (!R) {
        // Tile height: a tile costs its R * CW / 8 steps of 8 pixels plus a fixed share (the refill of its ring
        // slot is not hidden behind so few MMAs: about 8 steps' worth measured in plain TF32, 4 with the three times
        // longer steps of 3xTF32), and rows past the image edge are idle slots.  7 rows cover 7, 14, 28 and 56 pixel
        // high images exactly where 8 leave up to one slot in eight idle.  The taller tile on a tie.
        const int halves = diag ? 2 : 1, fixed = (mode3x && !diag) ? 4 : 8;
        long long best = -1;
        for (int cand : {8, 7, 4, 2, 1}) {
            if (cand > 1 && (2 * stage_bytes(cand) > 210 * 1024 || cand * halves > s->OH)) continue;
            const long long blocks = (s->OH + cand * halves - 1) / (cand * halves);
            const long long cost = blocks * ((long long)cand * (CW / 8) + fixed);   // diagonal: one MMA serves both halves
            if (best < 0 || cost < best) { best = cost; R = cand; }
        }
    }
    if (2 * stage_bytes(R) > 220 * 1024) return 1;
    if (strided && !opt(OPT_DW_R) && opt(OPT_DW_STRIDED) != 2) {
        // Few pixels per image leave tiles of one or two steps, whose fixed share dominates; below a fifth (3xTF32;
        // a seventh in plain TF32) of the steps doing work the split-K im2col kernel, whose tiles span images, is
        // faster (measured at 8x8x256 -> 4x4x512: 0.29 against 0.18 ms in 3xTF32, 0.131 against 0.126 ms in TF32).
        const int halves = diag ? 2 : 1, fixed = (mode3x && !diag) ? 4 : 8;
        long long cost = 0;
        for (int top = 0; top < s->OH; top += R * halves) cost += (long long)R * (CW / 8) + fixed;
        cost *= (s->OW + CW - 1) / CW;
        const double eff = (double)s->OH * s->OW / 8.0 / (double)(cost * halves);
        if (eff < (mode3x ? 0.2 : 0.15)) return 1;
    }
    int stages = (int)((220 * 1024) / stage_bytes(R));
    if (stages > 4) stages = 4;
    p.R = R; p.CW = CW; p.PW = PW;
    const int tile_rows = diag ? 2 * R : R;   // R = rows per half tile in the diagonal form
    p.row_blocks = (s->OH + tile_rows - 1) / tile_rows; p.col_blocks = (s->OW + CW - 1) / CW;
    p.tiles_per_img = p.row_blocks * p.col_blocks;
    const long long total = (long long)s->N * p.tiles_per_img;
    if (total > 2147483647LL) return 1;
    p.total_tiles = (int)total;
    int parts = sm_budget(c) / groups;
    if (parts < 1) parts = 1;
    if (parts > p.total_tiles) parts = p.total_tiles;
    if (per_image) {
        if (s->N > 65535 * 32 || deltaB) return 1;
        parts = s->N;
        p.per_image = 1;
    }
    p.parts = parts;
    p.stages = stages; p.mode3x = diag ? 3 : (stacked ? 2 : mode3x);
    p.idesc = make_idesc_tf32(kBM, stacked ? 2 * NT : NT, true, true);
    p.tmem_cols = pow2_cols(G * (stacked ? 2 * NT : NT));
    p.dy_tx = (uint32_t)R * CW * 128; p.dy_blk = (p.dy_tx + 1023) & ~1023u;
    p.x_tx = (uint32_t)R * PW * 128; p.x_blk = (p.x_tx + 1023) & ~1023u;
    p.sh = s->sh; p.sw = s->sw; p.nph = nph;
    {
        const uint32_t xph = (uint32_t)(NT / 32) * p.x_blk, xph_stride = stacked ? 2 * xph : xph;
        if (tgroups == 1) {
            for (int k = 0; k < nph; ++k) p.col_q0[k] = ph_qmin[k];
            for (int fw = 0; fw < s->FW; ++fw)
                p.tap_off16[fw] = (tap_k[fw] * xph_stride + (uint32_t)(tap_q[fw] - ph_qmin[tap_k[fw]]) * 128u) >> 4;
        } else {
            // stride 1, tap group tg: its tile starts at column fw_base - pw and tap fw_base + j starts j pixels later
            for (int tg = 0; tg < tgroups; ++tg) p.col_q0[tg] = tg * G - s->pw;
            for (int j = 0; j < 8; ++j) p.tap_off16[j] = (uint32_t)(j < G ? j : G - 1) * 8u;
        }
    }
    const size_t sizeW = (size_t)s->OC * s->FH * s->FW * s->IC;
    float* ws = nullptr;
    if (parts * nsub > 1 && !per_image) {
        int rc = get_workspace(c, stream, sizeW * parts * nsub * sizeof(float), &ws);
        if (rc) return rc;
        p.out = ws;
    } else {
        p.out = dW;
    }
    p.part_stride = sizeW;
    const size_t smem = (size_t)stages * stage_bytes(R) + (3 * stages + 2) * 8 + 1024;
    // fused bias gradient: per-CTA partial column sums, added in CTA order afterwards.  The cross-thread
    // sum borrows 16 KB of the operand ring.
    float* bias_parts = nullptr;
    if (deltaB && (size_t)stages * stage_bytes(R) >= 16384 && s->OC % 4 == 0) {
        int rc = get_workspace(c, stream, (size_t)parts * s->OC * sizeof(float), &bias_parts);
        if (rc) return rc;
        p.bias_out = bias_parts;
    }

    // X through one map per lattice phase [row phase][column phase]: rows phi, phi + sh, ... and columns psi, psi + sw, ...
    DwXMaps tmXs;
    CUtensorMap tmDY;
    int rc = 0;
    for (int phi = 0; phi < s->sh; ++phi)
        for (int k = 0; k < nph; ++k) {
            const int psi = ph_psi[k];
            cuuint64_t xd[4] = {(cuuint64_t)s->IC, (cuuint64_t)((s->IW - psi + s->sw - 1) / s->sw),
                                (cuuint64_t)((s->IH - phi + s->sh - 1) / s->sh), (cuuint64_t)s->N};
            cuuint64_t xs[3] = {(cuuint64_t)s->sw * s->IC * 4, (cuuint64_t)s->sh * s->IW * s->IC * 4, (cuuint64_t)s->IH * s->IW * s->IC * 4};
            cuuint32_t xbox[4] = {32, (cuuint32_t)PW, (cuuint32_t)R, 1};
            rc = make_tiled_map(&tmXs.m[phi * nph + k], X + ((size_t)phi * s->IW + psi) * s->IC, 4, xd, xs, xbox, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
            if (rc) return rc;
        }
    for (int i = s->sh * nph; i < 4; ++i) tmXs.m[i] = tmXs.m[0];
    cuuint64_t yd[4] = {(cuuint64_t)s->OC, (cuuint64_t)s->OW, (cuuint64_t)s->OH, (cuuint64_t)s->N};
    cuuint64_t ys[3] = {(cuuint64_t)s->OC * 4, (cuuint64_t)s->OW * s->OC * 4, (cuuint64_t)s->OH * s->OW * s->OC * 4};
    cuuint32_t ybox[4] = {32, (cuuint32_t)CW, (cuuint32_t)R, 1};
    rc = make_tiled_map(&tmDY, dY, 4, yd, ys, ybox, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;

    dim3 grid(parts, groups, 1);
    static bool attr_done = false;
    if (!attr_done) {
        dw_halo_set_attr<0, 0, 0>();
        dw_halo_set_attr<3, 1, 16>(); dw_halo_set_attr<3, 2, 16>(); dw_halo_set_attr<3, 4, 16>(); dw_halo_set_attr<3, 8, 16>();
        dw_halo_set_attr<3, 2, 8>(); dw_halo_set_attr<3, 4, 8>(); dw_halo_set_attr<3, 8, 8>();
        dw_halo_set_attr<3, 7, 16>(); dw_halo_set_attr<3, 7, 8>();
        dw_halo_set_attr<1, 2, 16>(); dw_halo_set_attr<1, 4, 16>(); dw_halo_set_attr<1, 8, 16>();
        dw_halo_set_attr<3, 2, 16, true>(); dw_halo_set_attr<3, 4, 16, true>(); dw_halo_set_attr<3, 8, 16, true>(); dw_halo_set_attr<3, 7, 16, true>();
        dw_halo_set_attr<3, 4, 8, true>(); dw_halo_set_attr<3, 8, 8, true>(); dw_halo_set_attr<3, 7, 8, true>();
        dw_halo_set_attr<4, 2, 16, true>(); dw_halo_set_attr<4, 4, 16, true>(); dw_halo_set_attr<4, 8, 16, true>();
        dw_halo_set_attr<4, 4, 8, true>(); dw_halo_set_attr<4, 8, 8, true>();
        dw_halo_set_attr<3, 2, 8, true>(); dw_halo_set_attr<4, 2, 8, true>(); dw_halo_set_attr<4, 7, 8, true>(); dw_halo_set_attr<4, 7, 16, true>();
        attr_done = true;
    }
#define DWH_LAUNCH(FW_, R_, CW_) do { if (!t_dry) conv_dw_halo_kernel<FW_, R_, CW_><<<grid, kDwHaloThreads, smem, stream>>>(tmXs, tmDY, p); } while (0)
#define DWH_LAUNCH_S(FW_, R_, CW_) do { if (!t_dry) conv_dw_halo_kernel<FW_, R_, CW_, true><<<grid, kDwHaloThreads, smem, stream>>>(tmXs, tmDY, p); } while (0)
    const bool st = G == 3 && !strided && opt(OPT_DW_STATIC) != 0;
    const bool st1 = s->FW == 1 && CW == 16 && opt(OPT_DW_STATIC) != 0;   // 1x1 (flat 16-column view; with a stride: one phase, start 0)
    const bool ss3 = s->FW == 3 && strided && opt(OPT_DW_STATIC) != 0, ss4 = s->FW == 4 && strided && opt(OPT_DW_STATIC) != 0;
    if (ss3 && R == 2 && CW == 16) DWH_LAUNCH_S(3, 2, 16);
    else if (ss3 && R == 4 && CW == 16) DWH_LAUNCH_S(3, 4, 16);
    else if (ss3 && R == 8 && CW == 16) DWH_LAUNCH_S(3, 8, 16);
    else if (ss3 && R == 7 && CW == 16) DWH_LAUNCH_S(3, 7, 16);
    else if (ss3 && R == 4 && CW == 8) DWH_LAUNCH_S(3, 4, 8);
    else if (ss3 && R == 8 && CW == 8) DWH_LAUNCH_S(3, 8, 8);
    else if (ss3 && R == 7 && CW == 8) DWH_LAUNCH_S(3, 7, 8);
    else if (ss4 && R == 2 && CW == 16) DWH_LAUNCH_S(4, 2, 16);
    else if (ss4 && R == 4 && CW == 16) DWH_LAUNCH_S(4, 4, 16);
    else if (ss4 && R == 8 && CW == 16) DWH_LAUNCH_S(4, 8, 16);
    else if (ss4 && R == 4 && CW == 8) DWH_LAUNCH_S(4, 4, 8);
    else if (ss4 && R == 8 && CW == 8) DWH_LAUNCH_S(4, 8, 8);
    else if (ss3 && R == 2 && CW == 8) DWH_LAUNCH_S(3, 2, 8);
    else if (ss4 && R == 2 && CW == 8) DWH_LAUNCH_S(4, 2, 8);
    else if (ss4 && R == 7 && CW == 8) DWH_LAUNCH_S(4, 7, 8);
    else if (ss4 && R == 7 && CW == 16) DWH_LAUNCH_S(4, 7, 16);
    else if (st && R == 1 && CW == 16) DWH_LAUNCH(3, 1, 16);
    else if (st && R == 2 && CW == 16) DWH_LAUNCH(3, 2, 16);
    else if (st && R == 4 && CW == 16) DWH_LAUNCH(3, 4, 16);
    else if (st && R == 8 && CW == 16) DWH_LAUNCH(3, 8, 16);
    else if (st && R == 2 && CW == 8) DWH_LAUNCH(3, 2, 8);
    else if (st && R == 4 && CW == 8) DWH_LAUNCH(3, 4, 8);
    else if (st && R == 8 && CW == 8) DWH_LAUNCH(3, 8, 8);
    else if (st && R == 7 && CW == 16) DWH_LAUNCH(3, 7, 16);
    else if (st && R == 7 && CW == 8) DWH_LAUNCH(3, 7, 8);
    else if (st1 && R == 2) DWH_LAUNCH(1, 2, 16);
    else if (st1 && R == 4) DWH_LAUNCH(1, 4, 16);
    else if (st1 && R == 8) DWH_LAUNCH(1, 8, 16);
    else DWH_LAUNCH(0, 0, 0);
#undef DWH_LAUNCH
#undef DWH_LAUNCH_S
    note_launch("dw_halo");
    snprintf(g_plan, sizeof(g_plan), "dw_halo%s%s NT=%d R=%d CW=%d stages=%d parts=%d groups=%d", diag ? " diagonal" : (stacked ? " stacked" : ""),
             strided ? (nph == 2 ? " strided 2 phases" : " strided") : (tgroups > 1 ? " tap groups of 3" : ""), NT, R, CW, stages, parts, groups);
    rc = check_launch("conv_dw_halo_kernel");
    if (rc || per_image) return rc;
    if (parts * nsub > 1) {
        const size_t n4 = sizeW / 4;
        if (!t_dry) launch_dw_reduce(ws, sizeW, parts * nsub, dW, n4, 0, stream, opt(OPT_DW_LANES));
        note_launch("dw_halo");
        rc = check_launch("dw_reduce_kernel");
    }
    if (!rc && bias_parts) {
        // the `parts` partial rows are a matrix whose columns want summing: 4 float4 columns x 64 row lanes per CTA
        const int cols4 = s->OC / 4, CT2 = cols4 < 4 ? cols4 : 4;
        if (!t_dry) field_sum_partial_kernel<<<dim3(1, (unsigned)((cols4 + CT2 - 1) / CT2)), kFieldSumThreads, 0, stream>>>(
            reinterpret_cast<const float4*>(bias_parts), parts, cols4, CT2, 64, reinterpret_cast<float4*>(deltaB));
        note_launch("dw_halo");
        rc = check_launch("field_sum_partial_kernel");
        if (bias_fused) *bias_fused = true;
    }
    return rc;
}

// Batched matrix products (the reference's Cuda_batchMatMul) on the convolution kernels: entry b of the batch is
// image b of a 1x1 convolution that has its own weights.  Dense matrices (row pitch = row length).  Returns 1 when
// the shape is outside what the tensor kernels take; the caller then runs its plain fp32 kernel.
//   form 0: C[b][N][M] = A[b][N][K] * B[b][K][M]      deltaX form, B read in place as an MN-major operand
//   form 1: C[b][N][M] = A[b][K][N]^T * B[b][K][M]    deltaW form, one CTA column per batch entry
//   form 2: C[b][N][M] = A[b][N][K] * B[b][M][K]^T    forward form
int launch_bmm_tensor(int form, const float* A, const float* B, float* C, int Batch, int N, int M, int K, cudaStream_t stream)
{
    if (cur_algo() == ALPHA_ALGO_SIMT) return 1;
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    ws_begin(c, stream);
    const int mode3x = cur_mode3x();
    if (form == 1) {
        // the K rows of A[b] and B[b] are the pixels of image b (16 per image row), OC = N, IC = M
        if (M % 32 != 0 || K % 16 != 0 || N % 4 != 0) return 1;
        AlphaConvShape s{};
        s.N = Batch; s.IH = s.OH = K / 16; s.IW = s.OW = 16; s.IC = M; s.OC = N;
        s.FH = s.FW = 1; s.sh = s.sw = 1; s.ph = s.pw = 0;
        return launch_dw_halo(c, &s, B, A, C, mode3x, stream, nullptr, nullptr, true);
    }
    if (K % 32 != 0 || N % 4 != 0 || M % 4 != 0) return 1;
    const int w = N % 8 == 0 ? 8 : 4;   // the N rows of A[b] as an image of w columns
    IgemmPlan pl{};
    pl.act = A; pl.aN = Batch; pl.aH = N / w; pl.aW = w; pl.aC = K;
    pl.FH = 1; pl.FW = 1; pl.sh = 1; pl.sw = 1; pl.pad_h = 0; pl.pad_w = 0;
    pl.out = C; pl.oH = N / w; pl.oW = w; pl.ncols = M;
    pl.W = B; pl.bias = nullptr; pl.kdim = K; pl.flip = false; pl.force = true;
    if (form == 2) { pl.wOC = Batch * M; pl.wIC = K; pl.b_mn = false; pl.w_img_rows = M; }
    else { pl.wOC = Batch * K; pl.wIC = M; pl.b_mn = true; pl.w_img_rows = K; }
    if ((long long)Batch * pl.w_img_rows > 2147483647LL) return 1;
    return launch_halo(c, pl, mode3x, stream);
}

// deltaW += sum of `part` split-K buffers of sizeW floats each (the reference's buf_summary).
int launch_buf_summary(cudaStream_t stream, const float* buf, float* deltaW, int part, size_t sizeW)
{
    const size_t n4 = sizeW / 4;
    if (!t_dry) launch_dw_reduce(buf, sizeW, part, deltaW, n4, 1, stream, opt(OPT_DW_LANES));
    note_launch("buf_summary");
    return check_launch("dw_reduce_kernel");
}


// ---- deltaW, split-K im2col kernel: plan and launch -----------------------------------------------
//
// One plan serves alpha_conv3d_deltaW (strides, and shapes the halo-tile kernel leaves) and
// alpha_conv3d_deltaW_noalloc; they differ only in where the split-K partial sums live.
struct DwSplitPlan {
    DwParams p;
    int groups = 0, n_tiles = 0, splits = 0, stages = 0;
    size_t sizeW = 0, smem = 0;
};

static int plan_dw_split(const AlphaConvShape* s, int mode3x, int sm_count, DwSplitPlan* out)
{
    DwSplitPlan pl;
    DwParams& p = pl.p;
    p = DwParams{};
    p.Npix = s->N * s->OH * s->OW;
    p.OHo = s->OH; p.OWo = s->OW; p.sh = s->sh; p.sw = s->sw; p.ph = s->ph; p.pw = s->pw;
    p.FH = s->FH; p.FW = s->FW; p.IC = s->IC; p.OC = s->OC;
    p.icb = s->IC / 32;
    p.MB = s->FH * s->FW * p.icb;
    int BN = ((s->OC + 31) / 32) * 32;
    if (BN > 256) BN = 256;
    p.BN = BN;
    const int MT = (p.MB + 3) / 4;
    int G = 512 / BN;  // accumulators of BN columns that fit the 512 tensor-memory columns
    if (G > MT) G = MT;
    const int groups = (MT + G - 1) / G;
    G = (MT + groups - 1) / groups;  // balance the groups
    p.G = G;
    p.KP = 32;
    p.tmem_cols = pow2_cols(G * BN);
    p.idesc = make_idesc_tf32(kBM, BN, true, true);
    p.mode3x = mode3x;
    const int n_tiles = (s->OC + BN - 1) / BN;
    p.total_chunks = (p.Npix + p.KP - 1) / p.KP;
    int splits = sm_count / (groups * n_tiles);
    if (splits < 1) splits = 1;
    if (splits > p.total_chunks) splits = p.total_chunks;
    p.chunks_per_split = (p.total_chunks + splits - 1) / splits;
    splits = (p.total_chunks + p.chunks_per_split - 1) / p.chunks_per_split;
    pl.sizeW = (size_t)s->OC * s->FH * s->FW * s->IC;
    const uint32_t blk = p.KP * 128;
    const uint32_t stage = (4 * blk + (BN / 32) * blk) * (mode3x ? 2 : 1);
    int stages = (int)((200u * 1024) / stage);
    if (stages > 6) stages = 6;
    if (stages < 1) return fail(ALPHA_E_ARG, "deltaW stage of %u bytes does not fit shared memory", stage);
    p.stages = stages;
    pl.smem = (size_t)stages * stage + (3 * stages + 2) * 8 + 1024;
    pl.groups = groups; pl.n_tiles = n_tiles; pl.splits = splits; pl.stages = stages;
    *out = pl;
    return ALPHA_OK;
}

// `partials` holds plan.splits * plan.sizeW floats when plan.splits > 1 and is not used otherwise.
static int launch_dw_split(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW, float* partials,
                           int* status, const DwSplitPlan& pl, cudaStream_t stream, const char* tag)
{
    DwParams p = pl.p;
    p.status = status;
    if (pl.splits > 1) { p.out = partials; p.split_stride = pl.sizeW; }
    else { p.out = deltaW; p.split_stride = 0; }
    CUtensorMap tmX, tmDY;
    int rc = make_im2col_map(&tmX, X, s->N, s->IH, s->IW, s->IC, s->FH, s->FW, s->sh, s->sw, s->ph, s->pw, 32, p.KP,
                             CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;
    cuuint64_t dd[2] = {(cuuint64_t)s->OC, (cuuint64_t)p.Npix};
    cuuint64_t ds[1] = {(cuuint64_t)s->OC * 4};
    cuuint32_t box[2] = {32, (cuuint32_t)p.KP};
    rc = make_tiled_map(&tmDY, deltaY, 2, dd, ds, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;
    dim3 grid(pl.groups, pl.n_tiles, pl.splits);
    if (!t_dry) conv_dw_kernel<<<grid, kIgemmThreads, pl.smem, stream>>>(tmX, tmDY, p);
    note_launch(tag);
    rc = check_launch("conv_dw_kernel");
    if (rc) return rc;
    if (pl.splits > 1) {
        const size_t n4 = pl.sizeW / 4;
        if (!t_dry) launch_dw_reduce(partials, pl.sizeW, pl.splits, deltaW, n4, 0, stream, opt(OPT_DW_LANES));
        note_launch(tag);
        rc = check_launch("dw_reduce_kernel");
    }
    return rc;
}

// ---- deltaW without any allocation ---------------------------------------------------------------
//
// Some hosts of this library must not allocate device memory at call time: a Java caller whose
// mempool has handed the whole card to the framework (Dragon-Alpha's engine owns every byte it
// could get and hands natives only addresses), a caller running inside a region where the CUDA
// allocator is off limits, or a real-time loop that cannot afford a cudaMalloc stall.  For them the
// split-K partials of deltaW live in this fixed array instead of the growable workspace.  Every
// GPU on which the library is loaded holds the array until the process exits.
constexpr size_t kNoAllocScratchBytes = 32ull << 20;  // 32 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchBytes / sizeof(float)];
static __device__ int g_noalloc_status;               // kernel status word of this entry point

struct NoAllocCtx {
    bool init = false;
    int sm_count = 0;
    float* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    int* status = nullptr;     // device address of g_noalloc_status on this device
};
static NoAllocCtx g_noalloc_ctx[64];

// Once per device, with that device current: resolves the device addresses of the two symbols.
// In host code the names g_noalloc_scratch / g_noalloc_status are only handles; a kernel must be
// given the addresses cudaGetSymbolAddress returns.
static int get_noalloc_ctx(NoAllocCtx** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(ALPHA_E_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    NoAllocCtx& c = g_noalloc_ctx[dev];
    if (!c.init) {
        int major = 0, sms = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        if (major != 10) return fail(ALPHA_E_DEVICE, "device %d is not sm_100; this library is built for sm_100a only", dev);
        int rc = load_driver_entry_points();
        if (rc) return rc;
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return fail(ALPHA_E_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        c.scratch = static_cast<float*>(p);
        p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_status);
        if (e != cudaSuccess || !p) return fail(ALPHA_E_CUDA, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
        c.status = static_cast<int*>(p);
        e = cudaFuncSetAttribute(conv_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        c.sm_count = sms;
        c.init = true;
    }
    *out = &c;
    return ALPHA_OK;
}

}  // namespace alpha

using namespace alpha;

// ---- Winograd F(2,3) forward (3x3, stride 1) ----------------------------------------------------
//
// Filter, input and output transforms run as separate memory-bound kernels around four 3x1
// tensor-core convolutions; the scratch (transformed filter, input and products, about
// 2|X| + 2|Y| + 4/3|W|) and the weight planes of the inner convolutions are carved from the
// stream's block one after the other.
static int forward_direct(DeviceCtx* c, const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                          float* Y, cudaStream_t stream, int algo, int act_on = 0, float act_k = 0.f);

static int launch_winograd(DeviceCtx* c, const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                           float* Y, cudaStream_t stream)
{
    if (s->FH != 3 || s->FW != 3 || s->sh != 1 || s->sw != 1)
        return fail(ALPHA_E_ARG, "Winograd F(2,3) applies to 3x3 stride-1 convolutions only");
    if (s->OW != s->IW + 2 * s->pw - 2) return fail(ALPHA_E_ARG, "Winograd F(2,3): OW does not match IW, pw");
    const int OWp = (s->OW + 1) / 2;
    const size_t nU = (size_t)4 * s->OC * 3 * s->IC;
    const size_t nV = (size_t)4 * s->N * s->IH * OWp * s->IC;
    const size_t nM = (size_t)4 * s->N * s->OH * OWp * s->OC;
    float* ws = nullptr;
    int rc0 = get_workspace(c, stream, (nU + nV + nM) * sizeof(float), &ws);
    if (rc0) return rc0;
    float *U = ws, *V = ws + nU, *M = ws + nU + nV;
    const int cap = c->sm_count * 16;
    auto blocks = [&](size_t n) { size_t b = (n + 255) / 256; return (unsigned)(b < (size_t)cap ? (b ? b : 1) : cap); };
    if (!t_dry) wino_filter_kernel<<<blocks((size_t)s->OC * 3 * s->IC / 4), 256, 0, stream>>>(W, U, s->OC, s->IC);
    if (!t_dry) wino_input_kernel<<<blocks(nV / 16), 256, 0, stream>>>(X, V, s->N, s->IH, s->IW, s->IC, OWp, s->pw);
    note_launch("winograd");
    int rc = check_launch("winograd transforms");
    if (rc) return rc;
    AlphaConvShape t = *s;
    t.IW = OWp; t.OW = OWp; t.FW = 1; t.pw = 0;  // 3x1 convolution over column pairs
    for (int k = 0; k < 4; ++k) {
        rc = forward_direct(c, &t, V + (size_t)k * (nV / 4), U + (size_t)k * (nU / 4), nullptr, M + (size_t)k * (nM / 4),
                            stream, ALPHA_ALGO_AUTO);
        if (rc) return rc;
    }
    if (!t_dry) wino_output_kernel<<<blocks(nM / 16), 256, 0, stream>>>(M, bias, Y, s->N, s->OH, s->OW, s->OC, OWp);
    note_launch("winograd");
    return check_launch("wino_output_kernel");
}

// ---- C ABI, layer 1 ----------------------------------------------------------------------------

extern "C" {

const char* alpha_conv_last_error(void) { return g_err; }
int alpha_conv_version(void) { return 100; }
int alpha_conv_set_math_mode(int mode)
{
    if (mode != ALPHA_MATH_3XTF32 && mode != ALPHA_MATH_TF32) return fail(ALPHA_E_ARG, "unknown math mode %d", mode);
    g_math.store(mode);
    return ALPHA_OK;
}
int alpha_conv_get_math_mode(void) { return g_math.load(); }
int alpha_conv_set_algo(int algo)
{
    if (algo < ALPHA_ALGO_AUTO || algo > ALPHA_ALGO_WINOGRAD) return fail(ALPHA_E_ARG, "unknown algo %d", algo);
    g_algo.store(algo);
    return ALPHA_OK;
}
int alpha_conv_get_algo(void) { return g_algo.load(); }
unsigned long long alpha_conv_launch_count(void) { return g_launches.load(); }
const char* alpha_conv_last_algo(void) { return g_last_algo; }
const char* alpha_conv_last_plan(void) { return g_plan; }

int alpha_conv_set_option(const char* name, int value)
{
    if (!name) return fail(ALPHA_E_ARG, "set_option: null name");
    if (!strncmp(name, "ALPHA_", 6)) name += 6;
    for (int i = 0; i < OPT_COUNT; ++i)
        if (!strcmp(name, kOptDefs[i].name)) {
            opt(static_cast<Opt>(i));   // seed the table from the environment first
            g_opt[i].store(value);
            return ALPHA_OK;
        }
    return fail(ALPHA_E_ARG, "set_option: unknown option %s", name);
}
int alpha_conv_get_option(const char* name, int* value)
{
    if (!name || !value) return fail(ALPHA_E_ARG, "get_option: null argument");
    if (!strncmp(name, "ALPHA_", 6)) name += 6;
    for (int i = 0; i < OPT_COUNT; ++i)
        if (!strcmp(name, kOptDefs[i].name)) { *value = opt(static_cast<Opt>(i)); return ALPHA_OK; }
    return fail(ALPHA_E_ARG, "get_option: unknown option %s", name);
}

int alpha_conv_set_workspace(alpha_stream_t stream_, void* ptr, size_t bytes)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    if (ptr && ((uintptr_t)ptr & 255)) return fail(ALPHA_E_ARG, "set_workspace: the block must be 256-byte aligned");
    cudaStream_t stream = (cudaStream_t)stream_;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx::Block& b = c->workspace[stream];
    if (b.base && !b.external) c->retired.push_back(DeviceCtx::Retired{b.base, b.bytes, nullptr, b.captured, stream});
    b = DeviceCtx::Block{};
    if (ptr) { b.base = static_cast<char*>(ptr); b.bytes = bytes; b.external = true; }
    return ALPHA_OK;
}

int alpha_conv_reserve_workspace(alpha_stream_t stream_, size_t bytes)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx::Block& b = c->workspace[stream];
    if (b.bytes >= bytes) return ALPHA_OK;
    rc = grow_block(c, stream, b, bytes);
    if (rc) return rc;
    // nothing of the old block is in use by a call in progress: its event can be recorded right away
    if (!c->retired.empty() && !c->retired.back().done && !c->retired.back().captured &&
        cudaEventCreateWithFlags(&c->retired.back().done, cudaEventDisableTiming) == cudaSuccess)
        cudaEventRecord(c->retired.back().done, stream);
    return ALPHA_OK;
}

int alpha_conv_release_workspace(void)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(g_mu);
    for (auto& kv : c->workspace)
        if (kv.second.base && !kv.second.external) cudaFree(kv.second.base);
    c->workspace.clear();
    for (DeviceCtx::Retired& r : c->retired) {
        if (r.done) cudaEventDestroy(r.done);
        cudaFree(r.ptr);
    }
    c->retired.clear();
    for (auto& kv : c->weights) {
        if (kv.second.ready) cudaEventDestroy(kv.second.ready);
        if (kv.second.ptr) cudaFree(kv.second.ptr);
    }
    c->weights.clear();
    return ALPHA_OK;
}

size_t alpha_conv_workspace_in_use(void)
{
    DeviceCtx* c;
    if (get_ctx(&c)) return 0;
    std::lock_guard<std::mutex> lock(g_mu);
    size_t total = 0;
    for (auto& kv : c->workspace) if (!kv.second.external) total += kv.second.bytes;
    for (DeviceCtx::Retired& r : c->retired) total += r.bytes;
    for (auto& kv : c->weights) total += kv.second.bytes;
    return total;
}

int alpha_conv_weight_cache(int enable)
{
    g_weight_cache.store(enable ? 1 : 0);
    return ALPHA_OK;
}

int alpha_conv_weights_updated(const float* W)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(g_mu);
    for (auto& kv : c->weights)
        if (!W || kv.first.W == W) kv.second.valid = false;
    return ALPHA_OK;
}

int alpha_conv_device_status(void)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int h = 0;
    e = cudaMemcpy(&h, c->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemcpy(status): %s", cudaGetErrorString(e));
    if (h != 0) {
        cudaMemset(c->status, 0, sizeof(int));
        fail(ALPHA_E_KERNEL, "a kernel left status %d (1 producer, 2 mma, 3 split, 4 epilogue wait ran out)", h);
    }
    return h;
}

int alpha_conv_debug_counters(unsigned long long* out, int n)
{
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    if (!c->prof) return fail(ALPHA_E_ARG, "cycle counters are off: set ALPHA_CONV_PROF=1 before the first call");
    if (n > kProfSlots) n = kProfSlots;
    cudaError_t e = cudaMemcpy(out, c->prof, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemcpy(counters): %s", cudaGetErrorString(e));
    return ALPHA_OK;
}

int alpha_conv3d_forward(const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                         float* Y, alpha_stream_t stream_)
{
    OpRange range("alpha_conv3d_forward");
    int rc = check_shape(s, X, W, Y);
    if (rc) return rc;
    if (bias && ((uintptr_t)bias & 15)) return fail(ALPHA_E_ARG, "bias must be 16-byte aligned");
    DeviceCtx* c;
    rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    ws_begin(c, stream);
    const int algo = cur_algo();
    if (algo == ALPHA_ALGO_WINOGRAD) return launch_winograd(c, s, X, W, bias, Y, stream);
    return forward_direct(c, s, X, W, bias, Y, stream, algo);
}

int alpha_conv_bias_grad(const float* deltaY, long long rows, int OC, float* deltaB, alpha_stream_t stream_)
{
    OpRange range("alpha_conv_bias_grad");
    if (!deltaY || !deltaB || rows <= 0 || OC <= 0) return fail(ALPHA_E_ARG, "bias_grad: null pointer or empty matrix");
    if (OC % 4 != 0) return fail(ALPHA_E_ARG, "bias_grad: OC must be a multiple of 4 (the engine pads channels to 4)");
    if (((uintptr_t)deltaY & 15) || ((uintptr_t)deltaB & 15)) return fail(ALPHA_E_ARG, "bias_grad: pointers must be 16-byte aligned");
    DeviceCtx* c;
    int rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    ws_begin(c, stream);
    const int cols4 = OC / 4;
    // first pass: up to 64 float4 columns (1 KB of a row) per CTA, the rest of the 256 threads as row lanes
    const int CT = cols4 < 64 ? cols4 : 64;
    const int RL = kFieldSumThreads / CT;
    const int gy = (cols4 + CT - 1) / CT;
    // enough CTAs to keep every SM's memory pipeline full, at least 8 * RL rows each
    long long gx = ((long long)c->sm_count * 4 + gy - 1) / gy;
    const long long by_rows = (rows + 8LL * RL - 1) / (8LL * RL);
    if (gx > by_rows) gx = by_rows;
    float* ws = nullptr;
    rc = get_workspace(c, stream, (size_t)gx * OC * sizeof(float), &ws);
    if (rc) return rc;
    if (!t_dry) field_sum_partial_kernel<<<dim3((unsigned)gx, (unsigned)gy), kFieldSumThreads, 0, stream>>>(
        reinterpret_cast<const float4*>(deltaY), rows, cols4, CT, RL, reinterpret_cast<float4*>(ws));
    note_launch("field_sum");
    rc = check_launch("field_sum_partial_kernel");
    if (rc) return rc;
    // the gx partial rows are again a matrix whose columns want summing: 4 float4 columns x 64 row lanes per CTA
    // (few rows, so the pass is bound by load latency: many lanes, few loads each)
    const int CT2 = cols4 < 4 ? cols4 : 4;
    const int RL2 = 64;
    if (!t_dry) field_sum_partial_kernel<<<dim3(1, (unsigned)((cols4 + CT2 - 1) / CT2)), kFieldSumThreads, 0, stream>>>(
        reinterpret_cast<const float4*>(ws), gx, cols4, CT2, RL2, reinterpret_cast<float4*>(deltaB));
    note_launch("field_sum");
    return check_launch("field_sum_partial_kernel");
}

int alpha_conv3d_forward_leakyRelu(const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                                   float k, float* Y, alpha_stream_t stream_)
{
    int rc = check_shape(s, X, W, Y);
    if (rc) return rc;
    if (bias && ((uintptr_t)bias & 15)) return fail(ALPHA_E_ARG, "bias must be 16-byte aligned");
    if (!(k == k)) return fail(ALPHA_E_ARG, "leakyRelu: slope is NaN");
    DeviceCtx* c;
    rc = get_ctx(&c);
    if (rc) return rc;
    int algo = cur_algo();
    if (algo == ALPHA_ALGO_WINOGRAD) algo = ALPHA_ALGO_AUTO;   // the Winograd output pass has no activation stage
    ws_begin(c, (cudaStream_t)stream_);
    return forward_direct(c, s, X, W, bias, Y, (cudaStream_t)stream_, algo, 1, k);
}

}  // extern "C"

static int forward_direct(DeviceCtx* c, const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                          float* Y, cudaStream_t stream, int algo, int act_on, float act_k)
{
    int rc;
    const bool tensor_ok = pick_kc(s->IC) != 0 && s->ph < 128 && s->pw < 128 && s->FH <= 256 && s->FW <= 256;
    if (algo == ALPHA_ALGO_TENSOR && !tensor_ok)
        return fail(ALPHA_E_ARG, "tensor path needs IC %% 8 == 0 (IC=%d)", s->IC);
    if (algo != ALPHA_ALGO_SIMT && tensor_ok) {
        IgemmPlan pl{};
        pl.act = X; pl.aN = s->N; pl.aH = s->IH; pl.aW = s->IW; pl.aC = s->IC;
        pl.FH = s->FH; pl.FW = s->FW; pl.sh = s->sh; pl.sw = s->sw; pl.pad_h = s->ph; pl.pad_w = s->pw;
        pl.out = Y; pl.oH = s->OH; pl.oW = s->OW; pl.ncols = s->OC;
        pl.W = W; pl.wOC = s->OC; pl.wIC = s->IC; pl.bias = bias; pl.act_on = act_on; pl.act_k = act_k;
        pl.b_mn = false; pl.flip = false; pl.kdim = s->IC;
        const int mode3x = cur_mode3x();
        if (tiny_image(s->OH, s->OW) && (s->FH > 1 || s->FW > 1) && patch_path_ok(s) && env_tile_mode() != 1) {
            rc = launch_patch_gemm(c, pl, mode3x, stream);
            if (rc != 1) return rc;
        }
        rc = launch_halo(c, pl, mode3x, stream);
        if (rc != 1) return rc;
        return launch_igemm(c, pl, mode3x, stream);
    }
    if (algo != ALPHA_ALGO_SIMT && patch_path_ok(s)) {
        IgemmPlan pl{};
        pl.act = X; pl.aN = s->N; pl.aH = s->IH; pl.aW = s->IW; pl.aC = s->IC;
        pl.FH = s->FH; pl.FW = s->FW; pl.sh = s->sh; pl.sw = s->sw; pl.pad_h = s->ph; pl.pad_w = s->pw;
        pl.out = Y; pl.oH = s->OH; pl.oW = s->OW; pl.ncols = s->OC;
        pl.W = W; pl.wOC = s->OC; pl.wIC = s->IC; pl.bias = bias; pl.act_on = act_on; pl.act_k = act_k;
        rc = launch_patch_gemm(c, pl, cur_mode3x(), stream);
        if (rc != 1) return rc;
    }
    const size_t total = (size_t)s->N * s->OH * s->OW * s->OC;
    if (!t_dry) conv_fwd_simt<<<simt_grid(total, c->sm_count), 256, 0, stream>>>(X, W, bias, Y, to_dev_shape(s), act_on, act_k);
    note_launch("simt");
    return check_launch("conv_fwd_simt");
}

extern "C" {

int alpha_conv3d_deltaX(const AlphaConvShape* s, const float* deltaY, const float* W, float* deltaX,
                        alpha_stream_t stream_)
{
    OpRange range("alpha_conv3d_deltaX");
    int rc = check_shape(s, deltaY, W, deltaX);
    if (rc) return rc;
    DeviceCtx* c;
    rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    ws_begin(c, stream);
    const int algo = cur_algo();
    const int pad_h = s->FH - 1 - s->ph, pad_w = s->FW - 1 - s->pw;
    const bool tensor_ok = s->sh == 1 && s->sw == 1 && pick_kc(s->OC) != 0 && pad_h >= 0 && pad_w >= 0 &&
                           pad_h < 128 && pad_w < 128 && s->IH == s->OH + s->FH - 1 - 2 * s->ph &&
                           s->IW == s->OW + s->FW - 1 - 2 * s->pw;
    if (algo == ALPHA_ALGO_TENSOR && !tensor_ok)
        return fail(ALPHA_E_ARG, "tensor deltaX path needs stride 1, OC %% 8 == 0 and padding < filter");
    if (algo != ALPHA_ALGO_SIMT && tensor_ok) {
        IgemmPlan pl{};
        pl.act = deltaY; pl.aN = s->N; pl.aH = s->OH; pl.aW = s->OW; pl.aC = s->OC;
        pl.FH = s->FH; pl.FW = s->FW; pl.sh = 1; pl.sw = 1; pl.pad_h = pad_h; pl.pad_w = pad_w;
        pl.out = deltaX; pl.oH = s->IH; pl.oW = s->IW; pl.ncols = s->IC;
        pl.W = W; pl.wOC = s->OC; pl.wIC = s->IC; pl.bias = nullptr;
        pl.b_mn = true; pl.flip = true; pl.kdim = s->OC;
        const int mode3x = cur_mode3x();
        if (env_tile_mode() != 1 && s->OC % 32 == 0 && taps_fit64(s) && opt(OPT_DX_TRANSPOSE)) {
            // deltaX as a forward conv over deltaY with Wt[ic][rotated tap][oc], built once per call
            const int taps = s->FH * s->FW;
            const size_t nW = (size_t)s->OC * taps * s->IC;
            float* ws = nullptr;
            bool fresh = true;
            const DeviceCtx::WeightKey wkey{W, WK_DX_S1, s->OC, s->IC, s->FH * 256 + s->FW, 0, mode3x};
            rc = weight_planes(c, stream, wkey, (mode3x ? 2 : 1) * nW * sizeof(float), &ws, &fresh);
            if (rc) return rc;
            IgemmPlan pt = pl;
            pt.W = ws; pt.W_lo = mode3x ? ws + nW : nullptr;
            pt.wOC = s->IC; pt.wIC = s->OC; pt.b_mn = false; pt.flip = false;
            if (fresh) {
                dim3 tg((s->IC + 31) / 32, (s->OC + 31) / 32, taps);
                TapMap map{};
                map.n = taps;
                for (int t = 0; t < taps; ++t) map.src[t] = taps - 1 - t;
                if (transforms_run()) transpose_weights_kernel<<<tg, 256, 0, stream>>>(W, ws, mode3x ? ws + nW : nullptr, s->OC, s->IC, taps, map, mode3x);
                note_launch("transpose_w");
                rc = check_launch("transpose_weights_kernel");
                if (rc) return rc;
                weight_planes_ready(c, stream, wkey);
            }
            if (!mode3x) pt.W_lo = nullptr;
            if (tiny_image(s->IH, s->IW) && (s->FH > 1 || s->FW > 1) && (long long)taps * s->OC <= 16384) {
                rc = launch_patch_gemm(c, pt, mode3x, stream);
                if (rc != 1) return rc;
            }
            rc = launch_halo(c, pt, mode3x, stream);
            if (rc != 1) return rc;
        }
        rc = launch_halo(c, pl, mode3x, stream);
        if (rc != 1) return rc;
        return launch_igemm(c, pl, cur_mode3x(), stream);
    }
    if (algo != ALPHA_ALGO_SIMT && (s->sh > 1 || s->sw > 1)) {
        rc = launch_dx_col2im(c, s, deltaY, W, deltaX, cur_mode3x(), stream);
        if (rc != 1) return rc;
        rc = launch_dx_phases(c, s, deltaY, W, deltaX, cur_mode3x(), stream);
        if (rc != 1) return rc;
    }
    const size_t total = (size_t)s->N * s->IH * s->IW * s->IC;
    if (!t_dry) conv_dx_simt<<<simt_grid(total, c->sm_count), 256, 0, stream>>>(deltaY, W, deltaX, to_dev_shape(s));
    note_launch("simt");
    return check_launch("conv_dx_simt");
}

int alpha_conv3d_deltaW(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW,
                        alpha_stream_t stream_)
{
    OpRange range("alpha_conv3d_deltaW");
    int rc = check_shape(s, X, deltaY, deltaW);
    if (rc) return rc;
    DeviceCtx* c;
    rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    ws_begin(c, stream);
    const int algo = cur_algo();
    const bool tensor_ok = (s->IC % 32 == 0) && s->ph < 128 && s->pw < 128 && s->FH <= 256 && s->FW <= 256;
    if (algo == ALPHA_ALGO_TENSOR && !tensor_ok)
        return fail(ALPHA_E_ARG, "tensor deltaW path needs IC %% 32 == 0 (IC=%d)", s->IC);
    if (algo != ALPHA_ALGO_SIMT && patch_path_ok(s) && env_tile_mode() != 1 &&
        (!tensor_ok || (s->OH * s->OW <= 9 && (s->FH > 1 || s->FW > 1)))) {
        // deltaW[oc][k] = sum over pixels of deltaY[pixel][oc] * A[pixel][k]: a 1x1 deltaW over the patch matrix
        float* A = nullptr;
        int K = 0, Kp = 0;
        const size_t M = (size_t)s->N * s->OH * s->OW;
        rc = make_patch_matrix(c, patch_shape_of(s), X, stream, &A, &K, &Kp,
                               (size_t)s->OC * ((s->FH * s->FW * s->IC + 31) / 32 * 32));
        if (rc) return rc;
        float* dWp = K == Kp ? deltaW : A + M * Kp;
        AlphaConvShape t = *s;
        t.IH = s->OH; t.IW = s->OW; t.IC = Kp; t.FH = 1; t.FW = 1; t.sh = 1; t.sw = 1; t.ph = 0; t.pw = 0;
        rc = launch_dw_halo(c, &t, A, deltaY, dWp, cur_mode3x(), stream);
        if (rc < 0) return rc;
        if (rc == 0) {
            if (K == Kp) return ALPHA_OK;
            const size_t total4 = (size_t)s->OC * (K / 4);
            size_t blocks = (total4 + 255) / 256;
            if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
            if (!t_dry) unpad_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dWp, deltaW, s->OC, K, Kp);
            note_launch("dw_patch");
            return check_launch("unpad_rows_kernel");
        }
    }
    if (algo == ALPHA_ALGO_SIMT || !tensor_ok) {
        const size_t total = (size_t)s->OC * s->FH * s->FW * s->IC;
        if (!t_dry) conv_dw_simt<<<(unsigned)total, 128, 0, stream>>>(X, deltaY, deltaW, to_dev_shape(s));
        note_launch("simt");
        return check_launch("conv_dw_simt");
    }

    const int mode3x = cur_mode3x();
    rc = launch_dw_halo(c, s, X, deltaY, deltaW, mode3x, stream);
    if (rc != 1) return rc;
    DwSplitPlan pl;
    rc = plan_dw_split(s, mode3x, sm_budget(c), &pl);
    if (rc) return rc;
    float* ws = nullptr;
    if (pl.splits > 1) {
        rc = get_workspace(c, stream, pl.sizeW * pl.splits * sizeof(float), &ws);
        if (rc) return rc;
    }
    return launch_dw_split(s, X, deltaY, deltaW, ws, c->status, pl, stream, "dw");
}

static int check_call_options(int math_mode, int algo)
{
    if (math_mode != -1 && math_mode != ALPHA_MATH_3XTF32 && math_mode != ALPHA_MATH_TF32)
        return fail(ALPHA_E_ARG, "unknown math mode %d (-1 = the process default)", math_mode);
    if (algo != -1 && (algo < ALPHA_ALGO_AUTO || algo > ALPHA_ALGO_WINOGRAD))
        return fail(ALPHA_E_ARG, "unknown algo %d (-1 = the process default)", algo);
    return ALPHA_OK;
}

int alpha_conv3d_forward_ex(const AlphaConvShape* s, const float* X, const float* W, const float* bias, float* Y,
                            int math_mode, int algo, alpha_stream_t stream)
{
    int rc = check_call_options(math_mode, algo);
    if (rc) return rc;
    CallOptions guard(math_mode, algo);
    return alpha_conv3d_forward(s, X, W, bias, Y, stream);
}

int alpha_conv3d_deltaX_ex(const AlphaConvShape* s, const float* deltaY, const float* W, float* deltaX, int math_mode,
                           int algo, alpha_stream_t stream)
{
    int rc = check_call_options(math_mode, algo);
    if (rc) return rc;
    CallOptions guard(math_mode, algo);
    return alpha_conv3d_deltaX(s, deltaY, W, deltaX, stream);
}

int alpha_conv3d_deltaW_ex(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW, int math_mode,
                           int algo, alpha_stream_t stream)
{
    int rc = check_call_options(math_mode, algo);
    if (rc) return rc;
    CallOptions guard(math_mode, algo);
    return alpha_conv3d_deltaW(s, X, deltaY, deltaW, stream);
}

// Runs operator `op` on placeholder activations with launches off, so that only its weight-side transform is
// sized (mode 3) or computed into the caller's block (mode 1).
static int run_weight_transform(const AlphaConvShape* s, int op, const float* W, void* prepared, size_t bytes, int mode,
                                alpha_stream_t stream, size_t* need)
{
    if (!s || (op != ALPHA_OP_FORWARD && op != ALPHA_OP_DELTAX)) return fail(ALPHA_E_ARG, "prepared weights exist for ALPHA_OP_FORWARD and ALPHA_OP_DELTAX");
    float* fake = reinterpret_cast<float*>(static_cast<uintptr_t>(1) << 31);
    const float* w = W ? W : reinterpret_cast<const float*>(static_cast<uintptr_t>(3) << 30);
    t_prep = PreparedHint{w, static_cast<float*>(prepared), bytes, mode, 0, false};
    t_dry = true;
    t_dry_cur = t_dry_peak = 0;
    const int rc = op == ALPHA_OP_FORWARD ? alpha_conv3d_forward(s, fake, w, nullptr, fake, stream)
                                          : alpha_conv3d_deltaX(s, fake, w, fake, stream);
    t_dry = false;
    if (need) *need = t_prep.seen ? t_prep.need : 0;
    t_prep = PreparedHint{};
    return rc;
}

int alpha_conv_prepared_weights_bytes(const AlphaConvShape* s, int op, size_t* bytes)
{
    if (!bytes) return fail(ALPHA_E_ARG, "prepared_weights_bytes: null argument");
    return run_weight_transform(s, op, nullptr, nullptr, 0, 3, nullptr, bytes);
}

int alpha_conv_prepare_weights(const AlphaConvShape* s, int op, const float* W, void* prepared, size_t bytes, alpha_stream_t stream)
{
    if (!W || ((uintptr_t)W & 15)) return fail(ALPHA_E_ARG, "prepare_weights: W is null or not 16-byte aligned");
    if (bytes && (!prepared || ((uintptr_t)prepared & 255))) return fail(ALPHA_E_ARG, "prepare_weights: the block must be 256-byte aligned");
    return run_weight_transform(s, op, W, prepared, bytes, 1, stream, nullptr);
}

int alpha_conv3d_forward_prepared(const AlphaConvShape* s, const float* X, const float* W, const void* prepared, size_t bytes,
                                  const float* bias, float* Y, alpha_stream_t stream)
{
    t_prep = PreparedHint{W, static_cast<float*>(const_cast<void*>(prepared)), bytes, prepared ? 2 : 0, 0, false};
    const int rc = alpha_conv3d_forward(s, X, W, bias, Y, stream);
    t_prep = PreparedHint{};
    return rc;
}

int alpha_conv3d_deltaX_prepared(const AlphaConvShape* s, const float* deltaY, const float* W, const void* prepared, size_t bytes,
                                 float* deltaX, alpha_stream_t stream)
{
    t_prep = PreparedHint{W, static_cast<float*>(const_cast<void*>(prepared)), bytes, prepared ? 2 : 0, 0, false};
    const int rc = alpha_conv3d_deltaX(s, deltaY, W, deltaX, stream);
    t_prep = PreparedHint{};
    return rc;
}

int alpha_conv_workspace_bytes(const AlphaConvShape* s, int op, size_t* bytes)
{
    if (!s || !bytes) return fail(ALPHA_E_ARG, "workspace_bytes: null argument");
    // the call itself, with launches and copies switched off and placeholder addresses: what it asks
    // get_workspace for is what it will ask for with real tensors
    float* fake = reinterpret_cast<float*>(static_cast<uintptr_t>(1) << 31);
    t_dry = true;
    t_dry_cur = t_dry_peak = 0;
    int rc;
    switch (op) {
    case ALPHA_OP_FORWARD: rc = alpha_conv3d_forward(s, fake, fake, nullptr, fake, nullptr); break;
    case ALPHA_OP_DELTAX: rc = alpha_conv3d_deltaX(s, fake, fake, fake, nullptr); break;
    case ALPHA_OP_DELTAW: rc = alpha_conv3d_deltaW(s, fake, fake, fake, nullptr); break;
    case ALPHA_OP_BIAS_GRAD: rc = alpha_conv_bias_grad(fake, (long long)s->N * s->OH * s->OW, s->OC, fake, nullptr); break;
    default: rc = fail(ALPHA_E_ARG, "workspace_bytes: unknown op %d", op);
    }
    t_dry = false;
    *bytes = t_dry_peak;
    return rc;
}

int alpha_conv3d_deltaW_bias(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW, float* deltaB,
                             alpha_stream_t stream_)
{
    if (!deltaB) return alpha_conv3d_deltaW(s, X, deltaY, deltaW, stream_);
    int rc = check_shape(s, X, deltaY, deltaW);
    if (rc) return rc;
    if ((uintptr_t)deltaB & 15) return fail(ALPHA_E_ARG, "deltaW_bias: deltaB must be 16-byte aligned");
    DeviceCtx* c;
    rc = get_ctx(&c);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    // the halo-tile kernel (stride 1, IC % 32 == 0, images larger than 3 x 3) sums the columns of the deltaY
    // tiles it stages anyway; every other shape runs the two passes one after the other
    const bool tensor_ok = (s->IC % 32 == 0) && s->ph < 128 && s->pw < 128 && s->FH <= 256 && s->FW <= 256;
    const bool patch = patch_path_ok(s) && env_tile_mode() != 1 && (!tensor_ok || (s->OH * s->OW <= 9 && (s->FH > 1 || s->FW > 1)));
    if (cur_algo() != ALPHA_ALGO_SIMT && tensor_ok && !patch) {
        ws_begin(c, stream);
        bool fused = false;
        rc = launch_dw_halo(c, s, X, deltaY, deltaW, cur_mode3x(), stream, deltaB, &fused);
        if (rc < 0) return rc;
        if (rc == 0 && fused) return ALPHA_OK;
        if (rc == 0) return alpha_conv_bias_grad(deltaY, (long long)s->N * s->OH * s->OW, s->OC, deltaB, stream_);
    }
    rc = alpha_conv3d_deltaW(s, X, deltaY, deltaW, stream_);
    if (rc) return rc;
    return alpha_conv_bias_grad(deltaY, (long long)s->N * s->OH * s->OW, s->OC, deltaB, stream_);
}

size_t alpha_conv3d_deltaW_noalloc_capacity(void) { return kNoAllocScratchBytes; }

int alpha_conv3d_deltaW_noalloc(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW,
                                alpha_stream_t stream_)
{
    int rc = check_shape(s, X, deltaY, deltaW);
    if (rc) return rc;
    if (s->IC % 32 != 0)
        return fail(ALPHA_E_ARG, "deltaW_noalloc runs the tensor-core kernel only: IC must be a multiple of 32 (IC=%d)", s->IC);
    if (s->ph >= 128 || s->pw >= 128 || s->FH > 256 || s->FW > 256)
        return fail(ALPHA_E_ARG, "deltaW_noalloc: the im2col tensor map takes padding < 128 and filters up to 256 x 256 "
                    "(ph=%d pw=%d FH=%d FW=%d)", s->ph, s->pw, s->FH, s->FW);
    NoAllocCtx* c;
    rc = get_noalloc_ctx(&c);
    if (rc) return rc;
    // The split-K im2col kernel with the plan alpha_conv3d_deltaW uses for it (plan_dw_split), the
    // partial sums in the fixed array instead of the growable workspace.
    DwSplitPlan pl;
    rc = plan_dw_split(s, cur_mode3x(), c->sm_count, &pl);
    if (rc) return rc;
    if (pl.splits > 1) {
        const size_t need = pl.sizeW * pl.splits * sizeof(float);
        if (need > kNoAllocScratchBytes)
            return fail(ALPHA_E_NOSCRATCH,
                        "deltaW_noalloc: %d split-K partials of %zu floats need %zu bytes, the fixed scratch holds %zu; "
                        "use alpha_conv3d_deltaW for this shape",
                        pl.splits, pl.sizeW, need, (size_t)kNoAllocScratchBytes);
    }
    return launch_dw_split(s, X, deltaY, deltaW, c->scratch, c->status, pl, (cudaStream_t)stream_, "dw_noalloc");
}

int alpha_conv3d_deltaW_noalloc_status(void)
{
    NoAllocCtx* c;
    int rc = get_noalloc_ctx(&c);
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int h = 0;
    e = cudaMemcpy(&h, c->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemcpy(status): %s", cudaGetErrorString(e));
    if (h != 0) {
        cudaMemset(c->status, 0, sizeof(int));
        fail(ALPHA_E_KERNEL, "the no-allocation deltaW kernel left status %d", h);
    }
    return h;
}

}  // extern "C"
