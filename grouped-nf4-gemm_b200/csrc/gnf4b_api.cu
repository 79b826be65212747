// C ABI of libgnf4b.so (see include/gnf4b.h): argument checks, launch planning, launches.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "stream_kernel.cuh"
#include "decode_kernel.cuh"
#include "tensor_kernel.cuh"
#include "tensor_fwd_kernel.cuh"
#include "ep_kernels.cuh"
#include "ffn_kernel.cuh"
#include "ep_peer.cuh"
#include "host_stage.cuh"
#include "gather_kernel.cuh"

namespace gnf4b {

// Scratch of gnf4b_gemm_grouped_noalloc.  In host code this name is only a stand-in for the
// device array; its device address comes from cudaGetSymbolAddress (noalloc_scratch below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[GNF4B_NOALLOC_SCRATCH_BYTES];

static thread_local char g_cuda_err[256] = "";

static int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", what, cudaGetErrorString(e));
    return GNF4B_ECUDA;
}

struct DevInfo {
    int sm_count = 0;
    int smem_optin = 0;
    bool ok = false;
};

static int device_info(DevInfo* out) {
    static std::mutex mu;
    static DevInfo cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return GNF4B_EINVAL;
    std::lock_guard<std::mutex> lk(mu);
    if (!cache[dev].ok) {
        e = cudaDeviceGetAttribute(&cache[dev].sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(SM count)");
        e = cudaDeviceGetAttribute(&cache[dev].smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(shared memory)");
        cache[dev].ok = true;
    }
    *out = cache[dev];
    return GNF4B_OK;
}

// Device address of g_noalloc_scratch on the current device, looked up once per device.
static int noalloc_scratch(void** out) {
    static std::mutex mu;
    static void* cache[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return GNF4B_EINVAL;
    std::lock_guard<std::mutex> lk(mu);
    if (!cache[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return cuda_fail(e, "cudaGetSymbolAddress(noalloc scratch)");
        cache[dev] = p;
    }
    *out = cache[dev];
    return GNF4B_OK;
}

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ------------------------------------------------------------------ planning
struct Plan {
    int path = 0;            // GNF4B_PATH_STREAM / GNF4B_PATH_TENSOR
    // stream path
    int split_k = 1;
    int chunk_bytes = 1024;
    int n_chunks = 1;
    int chunks_per_split = 1;
    int rows_cap = 1;
    int a_units_pad = 32;
    int au = 0;
    int g_cache = 0;
    int64_t n_tiles = 0;
    size_t counters_bytes = 0;
    size_t ws_bytes = 0;
};

static int check_shape(int fmt, int op, int x_dtype, int s_dtype, int64_t T, int32_t G, int32_t E,
                       int64_t N, int64_t K) {
    if (fmt != GNF4B_FMT_NF4 && fmt != GNF4B_FMT_MXFP4) return GNF4B_EINVAL;
    if (op != GNF4B_OP_FWD && op != GNF4B_OP_DGRAD) return GNF4B_EINVAL;
    if (x_dtype != GNF4B_X_BF16 && x_dtype != GNF4B_X_FP16) return GNF4B_EINVAL;
    if (fmt == GNF4B_FMT_NF4 && s_dtype != GNF4B_S_F32 && s_dtype != GNF4B_S_BF16) return GNF4B_EINVAL;
    if (fmt == GNF4B_FMT_MXFP4 && s_dtype != GNF4B_S_E8M0) return GNF4B_EINVAL;
    if (T < 0 || G < 0 || E <= 0 || N <= 0 || K <= 0) return GNF4B_ESHAPE;
    if (K % (fmt == GNF4B_FMT_NF4 ? 64 : 32)) return GNF4B_ESHAPE;
    if (T > INT32_MAX) return GNF4B_ETOOBIG;
    return GNF4B_OK;
}

// x_dtype < 0: not known (sizing calls).  The tensor kernels multiply bf16 x bf16: when the planner would
// pick them for fp16 activations it picks the streaming kernel instead, so the plan made here is the plan
// that launches and its scratch sizes are the ones the launch uses.
static int make_plan(int fmt, int op, int x_dtype, int64_t T, int32_t G, int64_t N, int64_t K, int32_t max_rows,
                     uint32_t flags, const DevInfo& di, Plan* p) {
    const uint32_t want = flags & GNF4B_PATH_MASK;
    const int forced_split = (int)((flags & GNF4B_SPLITK_MASK) >> GNF4B_SPLITK_SHIFT);
    int path = (int)want;
    if (path == GNF4B_PATH_AUTO) {
        // Streaming kernels while groups are a couple of rows on average (their per-element cost
        // grows with the rows of a group); tensor cores beyond that.  Without a host-known
        // maximum the mean T/G decides.
        const double mean_rows = G > 0 ? (double)T / G : 0.0;
        // Crossover in mean rows per group.  The decode kernel streams an expert's weights once per PAIR of
        // rows at about 2.0 TB/s (1.6 TB/s for rows shorter than 2048 columns); the tensor kernel pays a
        // fixed MMA-issue cost per (128-row tile, 64-column stage) whatever the rows: 5.6 ns (NF4, two MMAs
        // per k-step) or 3.85 ns (MXFP4) with all SMs busy.  Measured on B200: Qwen3 gate_up crosses at a
        // mean of 4.3 rows (model 3.9), Qwen3 down at 3.5 (3.5), gpt-oss gate_up at 2.4 (2.5).  Rows longer
        // than 3072 columns are streamed once per row, not per pair: fixed 1.5.
        double cross = 1.5;
        if (K <= 3072) {
            const double scale_bytes = (fmt == GNF4B_FMT_NF4) ? (double)(K / 64) * 4.0 : (double)(K / 32);
            // (NF4 rows of up to 1024 columns keep both rows of a pass as fp32: 1.85 TB/s)
            const double rate = K >= 2048 ? 2.0e6 : ((fmt == GNF4B_FMT_NF4 && K <= 1024) ? 1.85e6 : 1.6e6);
            const double t_pass = (double)N * ((double)(K / 2) + scale_bytes) / rate;   // us
            const double t_tensor = (double)ceil_div(N, 128) * (double)ceil_div(K, 64) * (fmt == GNF4B_FMT_NF4 ? 5.6e-3 : 3.85e-3);
            cross = std::min(4.0, std::max(2.0, 2.0 * (t_tensor / t_pass - 0.5)));
        }
        // (the decode kernel takes groups of up to 16 rows, two at a time; what decides is the mean: measured with
        // routed batches, a largest group of 9 at a mean of 2.3 rows is 115 us on it against 135 us on the tensor kernel)
        const bool small = (max_rows > 0) ? (max_rows <= 16 && mean_rows <= cross) : (mean_rows <= 1.5);
        path = (op == GNF4B_OP_DGRAD) ? GNF4B_PATH_TENSOR : (small ? GNF4B_PATH_STREAM : GNF4B_PATH_TENSOR);
        if (forced_split > 1 && op == GNF4B_OP_FWD) path = GNF4B_PATH_STREAM;
        if (x_dtype == GNF4B_X_FP16 && op == GNF4B_OP_FWD) path = GNF4B_PATH_STREAM;
    }
    if (path == GNF4B_PATH_STREAM && op == GNF4B_OP_DGRAD) return GNF4B_EUNSUPPORTED;
    p->path = path;
    if (path == GNF4B_PATH_TENSOR) return GNF4B_OK;

    const int64_t row_bytes = K / 2;
    const int unit = (fmt == GNF4B_FMT_NF4) ? 32 : 16;   // chunk granularity in bytes
    p->n_tiles = ceil_div(N, kSTileN);
    int S = 1;
    int chunk = kSRowPitch;
    if (forced_split > 1) {
        S = forced_split;
        const int64_t want_chunk = round_up(ceil_div(row_bytes, S), unit);
        chunk = (int)std::min<int64_t>(kSRowPitch, std::max<int64_t>(unit, want_chunk));
    } else if (forced_split == 0) {
        // starved grid: fewer than two items per SM, and at least 2048 elements per split
        const int64_t items = (int64_t)G * p->n_tiles;
        const int64_t full_chunks = ceil_div(row_bytes, kSRowPitch);
        if (items > 0 && items < 2 * (int64_t)di.sm_count && full_chunks > 1) {
            const int64_t wantS = ceil_div(4 * (int64_t)di.sm_count, items);
            while (S < wantS && S < 8 && S * 2 <= full_chunks) S *= 2;
        }
    }
    p->chunk_bytes = chunk;
    p->n_chunks = (int)ceil_div(row_bytes, chunk);
    p->chunks_per_split = (int)ceil_div(p->n_chunks, S);
    p->split_k = (int)ceil_div(p->n_chunks, p->chunks_per_split);   // no empty splits
    p->a_units_pad = (int)round_up(K / 32, 32);
    // the first g_cache groups' offsets and expert ids live in shared memory
    p->g_cache = (int)std::min<int64_t>(G, 1024);
    const int64_t fixed = (int64_t)kSTableBytes + (int64_t)kSStages * kSStageBytes + 256 +
                          (int64_t)(2 * p->g_cache + 1) * 4;
    const int64_t per_row = (int64_t)p->a_units_pad * 128;
    int64_t cap = (di.smem_optin - fixed) / per_row;
    if (cap < 1) return GNF4B_EUNSUPPORTED;
    cap = std::min<int64_t>(cap, kSRowsMax);
    if (max_rows > 0) cap = std::min<int64_t>(cap, max_rows);
    p->rows_cap = (int)cap;
    // decode specialisation: the host knows every group has at most one row, one K pass
    p->au = (max_rows == 1 && p->split_k == 1 && chunk == kSRowPitch) ? (K <= 2048 ? 2 : (K <= 3072 ? 3 : 0)) : 0;
    if (p->split_k > 1) {
        p->counters_bytes = (size_t)round_up((int64_t)G * p->n_tiles * 4, 256);
        p->ws_bytes = (size_t)p->split_k * (size_t)T * (size_t)N * 4;
    }
    return GNF4B_OK;
}

// cudaFuncSetAttribute is per device and not free; raise a kernel's dynamic shared-memory
// limit only when a launch needs more than was already granted on this device.
template <typename F>
static cudaError_t ensure_smem(F kfn, size_t smem, int* granted /*[64], zero-initialised*/) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    dev &= 63;
    if ((int)smem > granted[dev]) {
        e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        granted[dev] = (int)smem;
    }
    return cudaSuccess;
}

// ------------------------------------------------------------------ launches
template <int FMT, int SDT>
static cudaError_t launch_stream_au(const StreamArgs& sa, int au, int grid, size_t smem, cudaStream_t st) {
#define GNF4B_LAUNCH_AU(AUV)                                                                          \
    do {                                                                                              \
        auto kfn = stream_gemm_kernel<FMT, SDT, AUV>;                                                 \
        static int granted[64];                                                                       \
        cudaError_t e = ensure_smem(kfn, smem, granted);                                              \
        if (e != cudaSuccess) return e;                                                               \
        kfn<<<grid, kSThreads, smem, st>>>(sa);                                                       \
        return cudaGetLastError();                                                                    \
    } while (0)
    if (au == 2) GNF4B_LAUNCH_AU(2);
    if (au == 3) GNF4B_LAUNCH_AU(3);
    GNF4B_LAUNCH_AU(0);
#undef GNF4B_LAUNCH_AU
}

// Launch with programmatic stream serialization: the kernel may start while its predecessor in the stream is
// still running and must call pdl_wait() before it touches anything (reads or writes) the predecessor may use.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kfn)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kfn, static_cast<KArgs>(args)...);
}

template <int FMT, int SDT, int AUV, int RMV, int RW, int XF, int XA = 0, int CH = 0>
static cudaError_t launch_decode_one(const DecodeArgs& da, int grid, size_t smem, cudaStream_t st) {
    auto kfn = decode_gemv_kernel<FMT, SDT, AUV, RMV, RW, XF, XA, CH>;
    static int granted[64];
    cudaError_t e = ensure_smem(kfn, smem, granted);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(CH ? (kDChainWarps + 1) * 32 : decode_threads(RMV, AUV));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kfn, da);
}

// rw: weight rows of a stage per warp in flight (2 only with one activation row per pass and short rows).
// Form of the activations and of the table (XF of the kernel): fp32 activations while they fit the registers
// (AU <= 2), bf16 pairs beyond; MXFP4, whose codebook is exact in bf16, always takes the bf16-pair table with the
// mixed-precision FMA.
template <int FMT, int SDT>
static cudaError_t launch_decode_au(const DecodeArgs& da, int au, int rm, int rw, bool bf16_rows, int grid, size_t smem,
                                    cudaStream_t st) {
    constexpr int X1 = (FMT == GNF4B_FMT_MXFP4) ? 2 : 1;     // short rows
    constexpr int X0 = (FMT == GNF4B_FMT_MXFP4) ? 2 : 0;     // long rows, two activation rows per pass
    if (da.x_act) {
        // activation applied on load: the FFN's second GEMM, whose rows (the intermediate size) are short
        if (au > 3) return cudaErrorNotSupported;
        if (rm == 1 && rw == 2) {
            if (au <= 1) return launch_decode_one<FMT, SDT, 1, 1, 2, X1, 1>(da, grid, smem, st);
            if (au == 2) return launch_decode_one<FMT, SDT, 2, 1, 2, X1, 1>(da, grid, smem, st);
            return launch_decode_one<FMT, SDT, 3, 1, 2, X0, 1>(da, grid, smem, st);
        }
        if (rm == 2) {
            if (au <= 1) return launch_decode_one<FMT, SDT, 1, 2, 1, X0, 1>(da, grid, smem, st);
            if (au == 2) return launch_decode_one<FMT, SDT, 2, 2, 1, X0, 1>(da, grid, smem, st);
            return launch_decode_one<FMT, SDT, 3, 2, 1, X0, 1>(da, grid, smem, st);
        }
        return cudaErrorNotSupported;
    }
    if (rm == 1 && rw == 2) {
        if (au <= 1) return launch_decode_one<FMT, SDT, 1, 1, 2, X1>(da, grid, smem, st);
        if (au == 2) return launch_decode_one<FMT, SDT, 2, 1, 2, X1>(da, grid, smem, st);
        if (au == 3) return launch_decode_one<FMT, SDT, 3, 1, 2, X0>(da, grid, smem, st);
    }
    if (rm == 1) {
        if (au <= 1) return launch_decode_one<FMT, SDT, 1, 1, 1, X1>(da, grid, smem, st);
        if (au == 2) return launch_decode_one<FMT, SDT, 2, 1, 1, X1>(da, grid, smem, st);
        if (au == 3) return launch_decode_one<FMT, SDT, 3, 1, 1, X0>(da, grid, smem, st);
        // long rows: chained pairs of warps, each warp half of the row's units
        if (au <= 4) return launch_decode_one<FMT, SDT, 2, 1, 1, X0, 0, 1>(da, grid, smem, st);
        if (au <= 6) return launch_decode_one<FMT, SDT, 3, 1, 1, X0, 0, 1>(da, grid, smem, st);
        if (au <= 7) return launch_decode_one<FMT, SDT, 4, 1, 1, X0, 0, 1>(da, grid, smem, st);
    }
    if (rm == 2) {
        // rows of up to 1024 columns: both activation rows fit 64 registers of a lane as fp32, and an element then
        // costs its lookup and one FMA per row, without the two widening instructions per row of the bf16-pair form
        // (Qwen3 down, 768 columns: 15 % faster).  Longer rows keep bf16 pairs: splitting a row over two chained warps
        // so that each holds half of both rows as fp32 measured 8 % slower than the pairs at 2048 columns, and four
        // rows per pass (eight or seven warps, 128 registers of activations) twice as slow per pass as two.
        if (au <= 1) {
            if (bf16_rows) return launch_decode_one<FMT, SDT, 1, 2, 1, X0>(da, grid, smem, st);
            return launch_decode_one<FMT, SDT, 1, 2, 1, X1>(da, grid, smem, st);
        }
        if (au == 2) return launch_decode_one<FMT, SDT, 2, 2, 1, X0>(da, grid, smem, st);
        if (au == 3) return launch_decode_one<FMT, SDT, 3, 2, 1, X0>(da, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

template <int FMT, int SDT, int AU, int RW, int XF, int ACT>
static cudaError_t launch_ffn_one(const FfnArgs& fa, int grid, size_t smem, cudaStream_t st) {
    auto kfn = ffn_decode_kernel<FMT, SDT, AU, RW, XF, ACT>;
    static int granted[64];
    cudaError_t e = ensure_smem(kfn, smem, granted);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kFfnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kfn, fa);
}

template <int FMT, int SDT, int ACT>
static cudaError_t launch_ffn_au(const FfnArgs& fa, int au, int rw, int grid, size_t smem, cudaStream_t st) {
    constexpr int X1 = (FMT == GNF4B_FMT_MXFP4) ? 2 : 1;
    constexpr int X0 = (FMT == GNF4B_FMT_MXFP4) ? 2 : 0;
    if (rw == 2) {
        if (au <= 1) return launch_ffn_one<FMT, SDT, 1, 2, X1, ACT>(fa, grid, smem, st);
        if (au == 2) return launch_ffn_one<FMT, SDT, 2, 2, X0, ACT>(fa, grid, smem, st);
        if (au == 3) return launch_ffn_one<FMT, SDT, 3, 2, X0, ACT>(fa, grid, smem, st);
    } else {
        if (au <= 1) return launch_ffn_one<FMT, SDT, 1, 1, X1, ACT>(fa, grid, smem, st);
        if (au == 2) return launch_ffn_one<FMT, SDT, 2, 1, X0, ACT>(fa, grid, smem, st);
        if (au == 3) return launch_ffn_one<FMT, SDT, 3, 1, X0, ACT>(fa, grid, smem, st);
    }
    return cudaErrorInvalidValue;
}

static int align_class(const void* p, int64_t a, int64_t b) {
    const uint64_t v = (uint64_t)(uintptr_t)p | (uint64_t)a | (uint64_t)b;
    if ((v & 15) == 0) return 16;
    if ((v & 7) == 0) return 8;
    if ((v & 3) == 0) return 4;
    return 1;
}

// ------------------------------------------------------------------ small kernels
__global__ void offsets_kernel(const int32_t* sizes, int32_t G, int32_t* off) {
    // one warp, ordered scan: G is at most a few thousand
    __shared__ int32_t carry;
    if (threadIdx.x == 0) { carry = 0; off[0] = 0; }
    __syncwarp();
    for (int base = 0; base < G; base += 32) {
        const int g = base + threadIdx.x;
        int v = (g < G) ? sizes[g] : 0;
        if (v < 0) v = 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, o);
            if ((int)threadIdx.x >= o) v += t;
        }
        const int c = carry;
        if (g < G) off[g + 1] = c + v;
        __syncwarp();
        if (threadIdx.x == 31) carry = c + v;
        __syncwarp();
    }
}

template <int FMT, int SDT>
__global__ void dequant_kernel(const uint8_t* W, int64_t w_se, int64_t w_sn, const void* S, int64_t s_se,
                               int64_t s_sn, int32_t E, int64_t N, int64_t K, float* out) {
    const int64_t half = K / 2;
    const int64_t total = (int64_t)E * N * half;
    const int64_t blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = i % half;
        const int64_t r = i / half;
        const int64_t n = r % N, e = r / N;
        const uint32_t b = W[e * w_se + n * w_sn + j];
        const float2 p = byte_pair<FMT>(b);
        const float sc = load_scale<SDT>(S, e * s_se + n * s_sn + (2 * j) / blk);
        reinterpret_cast<float2*>(out)[(e * N + n) * half + j] = make_float2(p.x * sc, p.y * sc);
    }
}

}  // namespace gnf4b

using namespace gnf4b;

extern "C" {

int gnf4b_abi_version(void) { return GNF4B_ABI_VERSION; }


const char* gnf4b_strerror(int rc) {
    switch (rc) {
        case GNF4B_OK: return "ok";
        case GNF4B_EINVAL: return "invalid argument (enum, null or misaligned pointer, negative size)";
        case GNF4B_ESHAPE: return "shape violates the contract (K not a multiple of the quant block, N <= 0, ...)";
        case GNF4B_EWORKSPACE: return "workspace missing or smaller than gnf4b_workspace_bytes()";
        case GNF4B_ECUDA: return "a CUDA runtime call failed (gnf4b_last_cuda_error has the text)";
        case GNF4B_EUNSUPPORTED: return "this combination is not supported by the requested path";
        case GNF4B_ETOOBIG: return "a size exceeds a fixed maximum of this entry point";
        default: return "unknown gnf4b error";
    }
}

const char* gnf4b_last_cuda_error(void) { return g_cuda_err; }

int gnf4b_device_info(int32_t* sm_count, int32_t* smem_optin_bytes) {
    DevInfo di;
    int rc = device_info(&di);
    if (rc) return rc;
    if (sm_count) *sm_count = di.sm_count;
    if (smem_optin_bytes) *smem_optin_bytes = di.smem_optin;
    return GNF4B_OK;
}

size_t gnf4b_workspace_bytes(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K,
                             int32_t max_rows, uint32_t flags) {
    DevInfo di;
    if (device_info(&di)) return 0;
    // the call does not say which activation dtype will come: the larger of the two plans' needs
    size_t need = 0;
    for (int xdt : {GNF4B_X_BF16, GNF4B_X_FP16}) {
        Plan p;
        if (make_plan(fmt, op, xdt, T, G, N, K, max_rows, flags, di, &p) == GNF4B_OK)
            need = std::max(need, p.counters_bytes + p.ws_bytes);
    }
    return need;
}

int gnf4b_plan_split_k(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K, int32_t max_rows,
                       uint32_t flags) {
    DevInfo di;
    int rc = device_info(&di);
    if (rc) return rc;
    Plan p;
    rc = make_plan(fmt, op, GNF4B_X_BF16, T, G, N, K, max_rows, flags, di, &p);
    if (rc) return rc;
    return p.path == GNF4B_PATH_STREAM ? p.split_k : 1;
}

int gnf4b_gemm_grouped(int fmt, int op, const void* x, int x_dtype, int64_t T, const uint8_t* W,
                       int64_t w_stride_e, int64_t w_stride_n, const void* S, int s_dtype,
                       int64_t s_stride_e, int64_t s_stride_n, const int32_t* group_offsets,
                       const int32_t* expert_ids, int32_t G, int32_t E, int64_t N, int64_t K,
                       int32_t max_rows, void* out, void* workspace, size_t workspace_bytes,
                       int32_t* status_word, uint32_t flags, void* cuda_stream) {
    int rc = check_shape(fmt, op, x_dtype, s_dtype, T, G, E, N, K);
    if (rc) return rc;
    if (T == 0 || G == 0) return GNF4B_OK;
    if (!x || !W || !S || !group_offsets || !expert_ids || !out) return GNF4B_EINVAL;
    if (((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return GNF4B_EINVAL;
    if (w_stride_n < K / 2 || w_stride_e < 0 || s_stride_n < 0 || s_stride_e < 0) return GNF4B_EINVAL;
    DevInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    // activation applied while x is loaded: the decode kernel only
    const int x_act = (flags & GNF4B_FLAG_X_SILU_GLU) ? 1 : ((flags & GNF4B_FLAG_X_GPT_OSS_GLU) ? 2 : 0);
    if (x_act) {
        if (op != GNF4B_OP_FWD || x_dtype != GNF4B_X_BF16 || max_rows <= 0 || max_rows > 16) return GNF4B_EUNSUPPORTED;
        flags = (flags & ~(GNF4B_PATH_MASK | GNF4B_SPLITK_MASK)) | GNF4B_PATH_STREAM | (1u << GNF4B_SPLITK_SHIFT);
    }
    Plan p;
    rc = make_plan(fmt, op, x_dtype, T, G, N, K, max_rows, flags, di, &p);
    if (rc) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);

    GemmArgs g;
    g.x = x; g.W = W; g.S = S; g.off = group_offsets; g.eids = expert_ids; g.out = out;
    g.ws = nullptr; g.counters = nullptr; g.status = status_word;
    g.w_se = w_stride_e; g.w_sn = w_stride_n; g.s_se = s_stride_e; g.s_sn = s_stride_n;
    g.T = T; g.N = N; g.K = K; g.G = G; g.E = E; g.x_dtype = x_dtype; g.split_k = 1;

    if (p.path == GNF4B_PATH_TENSOR) {
        // forward: weight tile in tensor memory; dgrad (and GNF4B_FLAG_SMEM_OPERANDS): both operands
        // in shared memory
        rc = GNF4B_EUNSUPPORTED;
        if (op == GNF4B_OP_FWD && !(flags & GNF4B_FLAG_SMEM_OPERANDS))
            rc = launch_tensor_fwd(fmt, s_dtype, g, di.sm_count, di.smem_optin, align_class(W, w_stride_e, w_stride_n),
                                   (flags & GNF4B_FLAG_CTA_PAIR) != 0, st);
        if (rc == GNF4B_EUNSUPPORTED)      // dgrad, the ablation flag, or more groups than its table holds
            rc = launch_tensor(fmt, op, s_dtype, g, max_rows, di.sm_count, di.smem_optin,
                               align_class(W, w_stride_e, w_stride_n), st);
        if (rc == GNF4B_ECUDA) return cuda_fail(cudaGetLastError(), "tensor kernel launch");
        // A forward the tensor kernels decline for a reason the planner cannot see (no tensor-map encoder
        // in this driver, not enough shared memory) still has a CUDA kernel that takes it when the caller
        // left the choice to the planner.  Callers sized and cleared their scratch for the plan above, which
        // had none, so this second plan runs without split-K: it needs no scratch at all.
        const bool may_stream = rc == GNF4B_EUNSUPPORTED && op == GNF4B_OP_FWD &&
                                (flags & GNF4B_PATH_MASK) == GNF4B_PATH_AUTO;
        if (!may_stream) return rc;
        const uint32_t f2 = (flags & ~(GNF4B_PATH_MASK | GNF4B_SPLITK_MASK)) | GNF4B_PATH_STREAM | (1u << GNF4B_SPLITK_SHIFT);
        rc = make_plan(fmt, op, x_dtype, T, G, N, K, max_rows, f2, di, &p);
        if (rc) return rc;
    }

    if (p.split_k > 1) {
        if (!workspace || workspace_bytes < p.counters_bytes + p.ws_bytes) return GNF4B_EWORKSPACE;
        g.counters = reinterpret_cast<int32_t*>(workspace);
        g.ws = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + p.counters_bytes);
    }
    g.split_k = p.split_k;
    {
        // Decode kernel: at most 4 rows per group, contiguous 16-byte aligned rows and scale
        // rows, so a stage is two bulk copies (see decode_kernel.cuh).
        const int elt = (s_dtype == GNF4B_S_F32) ? 4 : (s_dtype == GNF4B_S_BF16 ? 2 : 1);
        const int64_t blk = (fmt == GNF4B_FMT_NF4) ? 64 : 32;
        const int64_t row_bytes = K / 2, srow = (K / blk) * elt;
        const bool contiguous = w_stride_n == row_bytes && s_stride_n == K / blk &&
                                (((uintptr_t)W | (uint64_t)w_stride_e) & 15) == 0 &&
                                (((uintptr_t)S | (uint64_t)(s_stride_e * elt)) & 15) == 0 && ((8 * srow) & 15) == 0;
        // rows of a group held in registers per pass: 1, or 2 with larger groups taken two rows at a
        // time (their weights are streamed once per pass; up to 8 passes)
        // (beyond K = 3072 one row at a time: two rows of 7168 columns do not fit a lane's registers)
        const int au_k = (int)ceil_div(K, 1024);
        const bool chunk_ok = max_rows >= 2 && max_rows <= 16 && G <= p.g_cache;
        const int rm = max_rows == 1 ? 1 : au_k > 3 ? (chunk_ok ? 1 : 0) : (max_rows == 2 || chunk_ok) ? 2 : 0;
        // long rows (one row per consumer warp and stage, 6 rows): the scale span of a stage and of the last,
        // shorter stage of a group must stay 16-byte aligned at that granularity
        const bool long_ok = au_k <= 3 || ((6 * srow) % 16 == 0 && (N % 6 == 0 || (((N % 6) * srow) % 16 == 0)));
        if (rm && long_ok && p.split_k == 1 && K <= 7168 && (N % 8) == 0 && contiguous &&
            x_dtype == GNF4B_X_BF16) {
            const int cw = decode_consumer_warps(rm, au_k);
            // two weight rows per warp in flight for one-row groups with short rows (see decode_kernel.cuh)
            const int rw = (rm == 1 && au_k <= 3 && !(flags & GNF4B_FLAG_DECODE_ONE_ROW)) ? 2 : 1;
            DecodeArgs da;
            da.g = g;
            // activation on load: room for the group's activated rows behind the group prefix
            // (long rows: the partial sums the chained pairs hand over, one set per ring stage, sit there instead)
            const int64_t h_bytes = x_act ? (int64_t)rm * K * 2 + 16 : (au_k > 3 ? (int64_t)kDMaxStages * kDChainPartialBytes + 16 : 0);
            const int64_t ring_room = (int64_t)di.smem_optin - (int64_t)decode_smem_bytes(0, 0, p.g_cache) - h_bytes;
            // a stage's scale span must stay 16-byte aligned: rows per stage in multiples of 4 when four scale
            // rows are, else of 8 (`contiguous` guarantees eight are)
            const int r_step = ((4 * srow) % 16 == 0) ? 4 : 8;
            int best_r;
            if (au_k > 3) {
                best_r = cw;                       // long_ok checked this granularity
                // two rows per pair and stage (half the hand-overs per byte) where twelve rows keep every span of a
                // stage -- the last, shorter one of a group too -- 16-byte aligned, and three such stages fit the ring
                if ((12 * srow) % 16 == 0 && (N % 12 == 0 || ((N % 12) * srow) % 16 == 0) &&
                    3 * (int64_t)12 * (row_bytes + srow) + 1024 <= ring_room &&
                    !(flags & GNF4B_FLAG_DECODE_ONE_ROW))
                    best_r = 2 * cw;
            } else {
                // rows per stage: up to 32 KiB of weight rows (at least rw per warp when three such stages fit the
                // ring), a whole number of rows per warp with rw = 2, and among the candidates the one that gives the
                // CTA with the most items the fewest rows (items are dealt out whole: with 768 items on 148 CTAs some
                // CTAs would stream 6 tiles and others 5); a small per-item charge keeps the stages from getting tiny
                int m = (int)std::max<int64_t>(1, std::min<int64_t>(4, 32768 / (cw * row_bytes)));
                if (m < rw && 3 * (int64_t)cw * rw * (row_bytes + srow) <= ring_room) m = rw;
                const int gran = (rw == 2 && m >= 2) ? cw * rw : r_step;
                const int r_hi = std::max(gran, (cw * m / gran) * gran);
                const int64_t groups_eff = std::max<int64_t>(1, std::min<int64_t>((int64_t)G * ((max_rows + rm - 1) / rm), T));
                best_r = r_hi;
                int64_t best_cost = INT64_MAX;
                for (int r = r_hi; r >= std::max(std::max(8, gran), r_hi / 2); r -= gran) {
                    const int64_t items = groups_eff * ceil_div(N, r);
                    const int64_t per_cta = ceil_div(items, std::min<int64_t>(di.sm_count, items));
                    const int64_t cost = per_cta * (r + 2);
                    if (cost < best_cost) { best_cost = cost; best_r = r; }
                }
            }
            da.rows_per_stage = best_r;
            da.tiles_per_group = (int32_t)ceil_div(N, da.rows_per_stage);
            da.row_bytes = (int32_t)row_bytes;
            da.scale_row_bytes = (int32_t)srow;
            da.slot_bytes = (int32_t)round_up((int64_t)da.rows_per_stage * (row_bytes + srow), 128);
            da.g_cache = p.g_cache;
            da.rows_per_pass = rm;
            da.row_chunks = (max_rows + rm - 1) / rm;
            // a list with more groups than rows is mostly empty (or padding) groups: walk only the ones that exist
            da.compact = (da.row_chunks > 1 || (((int64_t)G > T || (flags & GNF4B_FLAG_SPARSE_GROUPS)) && G <= p.g_cache)) ? 1 : 0;
            da.total_items = (int64_t)G * da.row_chunks * da.tiles_per_group;
            da.tables_ready = (flags & GNF4B_FLAG_TABLES_READY) ? 1 : 0;
            da.x_act = x_act;
            da.stages = (int32_t)std::min<int64_t>(kDMaxStages, ring_room / da.slot_bytes);
            const int dgrid = (int)std::min<int64_t>(di.sm_count, da.total_items);
            da.items_per_cta = (int32_t)(da.total_items / dgrid);
            da.items_extra = (int32_t)(da.total_items % dgrid);
            da.h_bytes = (int32_t)h_bytes;
            const size_t dsmem = decode_smem_bytes(da.slot_bytes, std::max(da.stages, 1), da.g_cache) + (size_t)h_bytes;
            if (da.stages >= 3 && da.total_items < (int64_t)1 << 31) {
                cudaError_t e;
                if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32)
                    e = launch_decode_au<GNF4B_FMT_NF4, GNF4B_S_F32>(da, au_k, rm, rw, (flags & GNF4B_FLAG_DECODE_BF16_ROWS) != 0, dgrid, dsmem, st);
                else if (fmt == GNF4B_FMT_NF4)
                    e = launch_decode_au<GNF4B_FMT_NF4, GNF4B_S_BF16>(da, au_k, rm, rw, (flags & GNF4B_FLAG_DECODE_BF16_ROWS) != 0, dgrid, dsmem, st);
                else
                    e = launch_decode_au<GNF4B_FMT_MXFP4, GNF4B_S_E8M0>(da, au_k, rm, rw, (flags & GNF4B_FLAG_DECODE_BF16_ROWS) != 0, dgrid, dsmem, st);
                if (e == cudaErrorNotSupported && x_act) return GNF4B_EUNSUPPORTED;
                if (e != cudaSuccess) return cuda_fail(e, "decode kernel launch");
                return GNF4B_OK;
            }
        }
    }
    if (x_act) return GNF4B_EUNSUPPORTED;       // the streaming kernel reads x as it is
    StreamArgs sa;
    sa.g = g;
    sa.n_tiles = (int32_t)p.n_tiles;
    sa.chunk_bytes = p.chunk_bytes;
    sa.n_chunks = p.n_chunks;
    sa.chunks_per_split = p.chunks_per_split;
    sa.rows_cap = p.rows_cap;
    sa.a_units_pad = p.a_units_pad;
    sa.w_align = align_class(W, w_stride_e, w_stride_n);
    sa.g_cache = p.g_cache;
    sa.total_items = (int64_t)G * p.n_tiles * p.split_k;
    const size_t smem = stream_smem_bytes(p.rows_cap, p.a_units_pad, p.g_cache);
    const int grid = (int)std::min<int64_t>(di.sm_count, sa.total_items);
    cudaError_t e;
    if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32)
        e = launch_stream_au<GNF4B_FMT_NF4, GNF4B_S_F32>(sa, p.au, grid, smem, st);
    else if (fmt == GNF4B_FMT_NF4)
        e = launch_stream_au<GNF4B_FMT_NF4, GNF4B_S_BF16>(sa, p.au, grid, smem, st);
    else
        e = launch_stream_au<GNF4B_FMT_MXFP4, GNF4B_S_E8M0>(sa, p.au, grid, smem, st);
    if (e != cudaSuccess) return cuda_fail(e, "stream kernel launch");
    return GNF4B_OK;
}

int gnf4b_gemm_grouped_noalloc(int fmt, int op, const void* x, int x_dtype, int64_t T, const uint8_t* W,
                               int64_t w_stride_e, int64_t w_stride_n, const void* S, int s_dtype,
                               int64_t s_stride_e, int64_t s_stride_n, const int32_t* group_offsets,
                               const int32_t* expert_ids, int32_t G, int32_t E, int64_t N, int64_t K,
                               int32_t max_rows, void* out, int32_t* status_word, uint32_t flags,
                               void* cuda_stream) {
    int rc = check_shape(fmt, op, x_dtype, s_dtype, T, G, E, N, K);
    if (rc) return rc;
    if (T == 0 || G == 0) return GNF4B_OK;
    DevInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    Plan p;
    rc = make_plan(fmt, op, x_dtype, T, G, N, K, max_rows, flags, di, &p);      // the plan that will launch
    if (rc) return rc;
    const size_t need = p.counters_bytes + p.ws_bytes;
    if (need > (size_t)GNF4B_NOALLOC_SCRATCH_BYTES) return GNF4B_ETOOBIG;
    void* scratch = nullptr;
    rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    if (p.counters_bytes) {
        // the arrival counters must start at zero whatever an earlier call left behind
        cudaError_t e = cudaMemsetAsync(scratch, 0, p.counters_bytes, reinterpret_cast<cudaStream_t>(cuda_stream));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(noalloc scratch)");
    }
    return gnf4b_gemm_grouped(fmt, op, x, x_dtype, T, W, w_stride_e, w_stride_n, S, s_dtype, s_stride_e, s_stride_n,
                              group_offsets, expert_ids, G, E, N, K, max_rows, out, scratch,
                              (size_t)GNF4B_NOALLOC_SCRATCH_BYTES, status_word, flags, cuda_stream);
}

// ---- host-buffer entry point -------------------------------------------------------------------
// Layout of the caller's device staging block (every piece 256-byte aligned):
//   [ planner workspace (worst case over routings) | offsets[G+1], ids[G], status | x | out ]
// tables, status and x are adjacent so that a small x travels in the same copy as the tables.
struct HostStaging {
    size_t ws = 0, tab = 0, x = 0, out = 0, total = 0;   // byte offsets; ws is at 0
    size_t ws_bytes = 0, tab_bytes = 0, x_bytes = 0, out_bytes = 0;
};

static int host_staging_layout(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K, uint32_t flags,
                               const DevInfo& di, HostStaging* h) {
    size_t worst = 0;
    const int32_t probes[2] = {1, -1};      // scratch exists only on the streaming path: both path choices,
    for (int32_t mr : probes) {             // and both activation dtypes (fp16 always streams)
        for (int xdt : {GNF4B_X_BF16, GNF4B_X_FP16}) {
            Plan p;
            const int rc = make_plan(fmt, op, xdt, T, G, N, K, mr, flags, di, &p);
            if (rc == GNF4B_OK) worst = std::max(worst, p.counters_bytes + p.ws_bytes);
            else if (rc != GNF4B_EUNSUPPORTED) return rc;
        }
    }
    const int64_t in_cols = (op == GNF4B_OP_FWD) ? K : N, out_cols = (op == GNF4B_OP_FWD) ? N : K;
    h->ws_bytes = worst;
    h->tab_bytes = (size_t)(2 * (int64_t)G + 2) * 4;
    h->x_bytes = (size_t)T * (size_t)in_cols * 2;
    h->out_bytes = (size_t)T * (size_t)out_cols * 2;
    h->tab = (size_t)round_up((int64_t)h->ws_bytes, 256);
    h->x = h->tab + (size_t)round_up((int64_t)h->tab_bytes, 256);
    h->out = h->x + (size_t)round_up((int64_t)h->x_bytes, 256);
    h->total = h->out + (size_t)round_up((int64_t)h->out_bytes, 256);
    return GNF4B_OK;
}

static constexpr size_t kHostPinnedBytes = 64u << 10;

// The calling thread's pinned block: [ in: group tables, and x when it fits | out: the result of a small call |
// tail: sequence number, status word ].  Pinned, portable and mapped: the GPU reads and writes it directly on the
// small-call path (host_stage.cuh).  Freed when the thread ends.
struct PinnedBlock {
    unsigned char* p = nullptr;
    unsigned char* dev = nullptr;          // the block as the current device addresses it
    uint32_t seq = 0;
    unsigned char* out() const { return p + kHostPinnedBytes; }
    volatile uint32_t* tail() const { return reinterpret_cast<volatile uint32_t*>(p + 2 * kHostPinnedBytes); }
    ~PinnedBlock() { if (p) cudaFreeHost(p); }
};

static PinnedBlock& thread_pinned_block() {
    static thread_local PinnedBlock pin;
    return pin;
}

static cudaError_t ensure_pinned_block(PinnedBlock& pin) {
    if (pin.p) return cudaSuccess;
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&pin.p), 2 * kHostPinnedBytes + 256,
                                  cudaHostAllocPortable | cudaHostAllocMapped);
    if (e != cudaSuccess) { pin.p = nullptr; return e; }
    void* d = nullptr;
    // with unified addressing the device address of mapped pinned memory is the host address; asked for anyway
    pin.dev = (cudaHostGetDevicePointer(&d, pin.p, 0) == cudaSuccess && d) ? static_cast<unsigned char*>(d) : nullptr;
    if (!pin.dev) (void)cudaGetLastError();
    pin.tail()[0] = 0;
    return cudaSuccess;
}

// A small call's way in and out without the copy engines (host_stage.cuh).  stage_in: the first `in_bytes` of the
// pinned block -> dst on the device, plus up to two spans zeroed.  stage_out + wait: src on the device -> the block's
// out area, then the host thread polls the sequence number (bounded: after 50 ms it falls back to a stream
// synchronise, which also surfaces a launch that failed).
static cudaError_t host_stage_in(PinnedBlock& pin, void* dst, size_t in_bytes, void* zero_a, size_t zero_a_bytes,
                                 void* zero_b, size_t zero_b_bytes, cudaStream_t st) {
    return launch_pdl(host_stage_in_kernel, 1u, (unsigned)kHostStageThreads, st, reinterpret_cast<const uint4*>(pin.dev),
                      static_cast<uint4*>(dst), (int32_t)(in_bytes / 16), static_cast<uint4*>(zero_a),
                      (int32_t)(zero_a_bytes / 16), static_cast<uint4*>(zero_b), (int32_t)(zero_b_bytes / 16));
}

static int host_stage_out_wait(PinnedBlock& pin, const void* src, size_t out_bytes, const int32_t* d_status, void* out_host,
                               int32_t* status_host, cudaStream_t st) {
    const uint32_t seq = ++pin.seq ? pin.seq : ++pin.seq;          // never 0
    cudaError_t e = launch_pdl(host_stage_out_kernel, 1u, (unsigned)kHostStageThreads, st, static_cast<const uint4*>(src),
                               reinterpret_cast<uint4*>(pin.dev + kHostPinnedBytes), (int32_t)(out_bytes / 16), d_status,
                               reinterpret_cast<volatile uint32_t*>(pin.dev + 2 * kHostPinnedBytes), seq);
    if (e != cudaSuccess) { cudaStreamSynchronize(st); return cuda_fail(e, "host_stage_out launch"); }
    volatile uint32_t* tail = pin.tail();
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t spins = 0;
    while (tail[0] != seq) {
        if ((++spins & 1023u) == 0 &&
            std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(50)) {
            e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
            if (tail[0] != seq) return cuda_fail(cudaErrorUnknown, "host_stage_out: result not delivered");
            break;
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    std::memcpy(out_host, pin.out(), out_bytes);
    if (status_host) *status_host = (int32_t)tail[1];
    return GNF4B_OK;
}

size_t gnf4b_host_staging_bytes(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K, uint32_t flags) {
    if (check_shape(fmt, op, GNF4B_X_BF16, fmt == GNF4B_FMT_NF4 ? GNF4B_S_F32 : GNF4B_S_E8M0, T, G, 1, N, K)) return 0;
    DevInfo di;
    if (device_info(&di)) return 0;
    HostStaging h;
    if (host_staging_layout(fmt, op, T, G, N, K, flags, di, &h)) return 0;
    return h.total;
}

int gnf4b_gemm_grouped_host(int fmt, int op, const void* x_host, int x_dtype, int64_t T, const uint8_t* W,
                            int64_t w_stride_e, int64_t w_stride_n, const void* S, int s_dtype,
                            int64_t s_stride_e, int64_t s_stride_n, const int32_t* sizes_host,
                            const int32_t* expert_ids_host, int32_t G, int32_t E, int64_t N, int64_t K,
                            void* out_host, void* staging, size_t staging_bytes, int32_t* status_host,
                            uint32_t flags, void* cuda_stream) {
    int rc = check_shape(fmt, op, x_dtype, s_dtype, T, G, E, N, K);
    if (rc) return rc;
    if (status_host) *status_host = 0;
    if (G > 0 && (!sizes_host || !expert_ids_host)) return GNF4B_EINVAL;
    int64_t total = 0;
    int32_t max_rows = 0;
    for (int32_t g = 0; g < G; ++g) {
        const int32_t n = sizes_host[g], e = expert_ids_host[g];
        if (n < 0 || (e != GNF4B_PAD_EXPERT && (e < 0 || e >= E))) return GNF4B_EINVAL;
        total += n;
        max_rows = std::max(max_rows, n);
    }
    if (total != T) return GNF4B_EINVAL;
    if (T == 0 || G == 0) return GNF4B_OK;
    if (!x_host || !out_host || !staging || ((uintptr_t)staging & 255)) return GNF4B_EINVAL;
    DevInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    HostStaging h;
    rc = host_staging_layout(fmt, op, T, G, N, K, flags, di, &h);
    if (rc) return rc;
    if (staging_bytes < h.total) return GNF4B_EWORKSPACE;
    Plan p;
    rc = make_plan(fmt, op, x_dtype, T, G, N, K, max_rows, flags, di, &p);      // the plan that will launch
    if (rc) return rc;

    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    unsigned char* base = static_cast<unsigned char*>(staging);
    int32_t* d_off = reinterpret_cast<int32_t*>(base + h.tab);
    int32_t* d_ids = d_off + (G + 1);
    int32_t* d_status = d_ids + G;
    void* d_x = base + h.x;
    void* d_out = base + h.out;
    cudaError_t e;

    PinnedBlock& pin = thread_pinned_block();
    e = ensure_pinned_block(pin);
    if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc(pinned block)");
    const size_t tab_span = h.x - h.tab;                 // tables + status, padded up to where x starts
    const bool tab_fits = tab_span <= kHostPinnedBytes;
    const bool x_rides = tab_fits && tab_span + h.x_bytes <= kHostPinnedBytes;
    // small call: in and out through the pinned block by two small kernels instead of the copy engines
    const bool direct = x_rides && pin.dev && h.out_bytes <= kHostPinnedBytes && h.out_bytes % 16 == 0 &&
                        !(flags & GNF4B_FLAG_HOST_COPIES);
    std::vector<int32_t> big_tab;                        // only for G beyond the pinned block
    int32_t* t = tab_fits ? reinterpret_cast<int32_t*>(pin.p) : (big_tab.resize(2 * (size_t)G + 2), big_tab.data());
    t[0] = 0;
    for (int32_t g = 0; g < G; ++g) t[g + 1] = t[g] + sizes_host[g];
    std::memcpy(t + G + 1, expert_ids_host, (size_t)G * 4);
    t[2 * (size_t)G + 1] = 0;                            // the status word starts clear
    if (direct) {
        std::memcpy(pin.p + tab_span, x_host, h.x_bytes);
        e = host_stage_in(pin, d_off, tab_span + h.x_bytes, base, p.counters_bytes, nullptr, 0, st);
        if (e != cudaSuccess) return cuda_fail(e, "host_stage_in launch");
        // the tables come from the kernel launched just before: not "ready" in the decode kernel's sense
        rc = gnf4b_gemm_grouped(fmt, op, d_x, x_dtype, T, W, w_stride_e, w_stride_n, S, s_dtype, s_stride_e, s_stride_n,
                                d_off, d_ids, G, E, N, K, max_rows, d_out, h.ws_bytes ? base : nullptr, h.ws_bytes,
                                d_status, flags & ~GNF4B_FLAG_TABLES_READY, cuda_stream);
        if (rc) { cudaStreamSynchronize(st); return rc; }
        return host_stage_out_wait(pin, d_out, h.out_bytes, d_status, out_host, status_host, st);
    }
    if (x_rides) {
        std::memcpy(pin.p + tab_span, x_host, h.x_bytes);
        e = cudaMemcpyAsync(d_off, pin.p, tab_span + h.x_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(tables + x)");
    } else {
        e = cudaMemcpyAsync(d_off, t, h.tab_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(tables)");
        e = cudaMemcpyAsync(d_x, x_host, h.x_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(x)");
    }
    if (p.counters_bytes) {
        e = cudaMemsetAsync(base, 0, p.counters_bytes, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(arrival counters)");
    }
    // the tables were uploaded by the copy above: ready when the kernel starts
    rc = gnf4b_gemm_grouped(fmt, op, d_x, x_dtype, T, W, w_stride_e, w_stride_n, S, s_dtype, s_stride_e, s_stride_n,
                            d_off, d_ids, G, E, N, K, max_rows, d_out, h.ws_bytes ? base : nullptr, h.ws_bytes,
                            d_status, flags | GNF4B_FLAG_TABLES_READY, cuda_stream);
    if (rc) { cudaStreamSynchronize(st); return rc; }    // the copies above read host memory: let them finish
    e = cudaMemcpyAsync(out_host, d_out, h.out_bytes, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) { cudaStreamSynchronize(st); return cuda_fail(e, "cudaMemcpyAsync(out)"); }
    if (status_host) {
        e = cudaMemcpyAsync(status_host, d_status, 4, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) { cudaStreamSynchronize(st); return cuda_fail(e, "cudaMemcpyAsync(status)"); }
    }
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return GNF4B_OK;
}

// ---- host-buffer expert FFN: one round trip around gnf4b_ffn_grouped -----------------------------------------
// Staging: [ workspace of gnf4b_ffn_grouped (worst case over routings) | offsets, ids, status | x | out ]
struct FfnStaging {
    size_t tab = 0, x = 0, out = 0, total = 0;
    size_t ws_bytes = 0, tab_bytes = 0, x_bytes = 0, out_bytes = 0;
};

static int ffn_check(int fmt, int x_dtype, int s_dtype, int64_t T, int32_t G, int32_t E, int64_t N_gu, int64_t K_gu,
                     int64_t N_dn) {
    int rc = check_shape(fmt, GNF4B_OP_FWD, x_dtype, s_dtype, T, G, E, N_gu, K_gu);
    if (rc) return rc;
    if (x_dtype != GNF4B_X_BF16) return GNF4B_EUNSUPPORTED;      // the GLU kernel writes bf16
    if (N_gu % 2) return GNF4B_ESHAPE;
    return check_shape(fmt, GNF4B_OP_FWD, x_dtype, s_dtype, T, G, E, N_dn, N_gu / 2);
}

int gnf4b_build_offsets(const int32_t* sizes, int32_t G, int32_t* group_offsets, void* cuda_stream) {
    if (G < 0 || !group_offsets || (G > 0 && !sizes)) return GNF4B_EINVAL;
    offsets_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(sizes, G, group_offsets);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "offsets kernel launch");
    return GNF4B_OK;
}

int gnf4b_upload_i32(const int32_t* host_src, int32_t* device_dst, int64_t n, void* cuda_stream) {
    if (n < 0 || (n > 0 && (!host_src || !device_dst))) return GNF4B_EINVAL;
    if (n == 0) return GNF4B_OK;
    cudaError_t e = cudaMemcpyAsync(device_dst, host_src, (size_t)n * 4, cudaMemcpyHostToDevice,
                                    reinterpret_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(group tables)");
    return GNF4B_OK;
}

int gnf4b_silu_glu(const void* gate_up, int64_t rows, int64_t h, void* out, void* cuda_stream) {
    if (rows < 0 || h <= 0 || (rows > 0 && (!gate_up || !out))) return GNF4B_EINVAL;
    if (rows == 0) return GNF4B_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    const bool vec = (h % 8) == 0 && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int64_t work = rows * (vec ? h / 8 : h);
    const int grid = (int)std::min<int64_t>(ceil_div(work, 256), 148 * 16);
    cudaError_t e = vec ? launch_pdl(silu_glu_kernel<8>, (unsigned)grid, 256u, st, static_cast<const uint16_t*>(gate_up), rows, h,
                                     static_cast<uint16_t*>(out))
                        : launch_pdl(silu_glu_kernel<1>, (unsigned)grid, 256u, st, static_cast<const uint16_t*>(gate_up), rows, h,
                                     static_cast<uint16_t*>(out));
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "silu_glu launch");
}

int gnf4b_glu_gpt_oss(const void* gate_up, int64_t rows, int64_t h, const void* bias, const int32_t* row_expert,
                      void* out, void* cuda_stream) {
    if (rows < 0 || h <= 0 || (rows > 0 && (!gate_up || !out)) || (bias && !row_expert)) return GNF4B_EINVAL;
    if (rows == 0) return GNF4B_OK;
    if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(bias)) & 3) return GNF4B_EINVAL;
    const int grid = (int)std::min<int64_t>(ceil_div(rows * h, 256), 148 * 16);
    glu_gpt_oss_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint16_t*>(gate_up), rows, h, static_cast<const uint16_t*>(bias), row_expert,
        static_cast<uint16_t*>(out));
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "glu_gpt_oss launch");
}

// ---- expert FFN on device pointers: one fused launch for one-row groups, three launches otherwise ----------
// Workspace: [ counters (G + 1) int32 | gate_up bf16 [T, N_gu] | h bf16 [T, N_gu / 2] | GEMM scratch ]
struct FfnWs {
    size_t counters = 0, gu = 0, h = 0, gemm = 0, total = 0, gemm_bytes = 0, gemm_counters = 0;
};

static int ffn_ws_layout(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn, int32_t max_rows,
                         uint32_t flags, const DevInfo& di, FfnWs* w) {
    auto up = [](size_t v) { return (size_t)round_up((int64_t)v, 256); };
    size_t gemm = 0, gemm_counters = 0;
    for (int xdt : {GNF4B_X_BF16}) {
        Plan a, b;
        int rc = make_plan(fmt, GNF4B_OP_FWD, xdt, T, G, N_gu, K_gu, max_rows, flags & GNF4B_PATH_MASK, di, &a);
        if (rc) return rc;
        rc = make_plan(fmt, GNF4B_OP_FWD, xdt, T, G, N_dn, N_gu / 2, max_rows, flags & GNF4B_PATH_MASK, di, &b);
        if (rc) return rc;
        gemm = std::max(gemm, std::max(a.counters_bytes + a.ws_bytes, b.counters_bytes + b.ws_bytes));
        gemm_counters = std::max(gemm_counters, std::max(a.counters_bytes, b.counters_bytes));
    }
    w->counters = 0;
    w->gu = up((size_t)(G + 1) * 4);
    w->h = w->gu + up((size_t)T * (size_t)N_gu * 2);
    w->gemm = w->h + up((size_t)T * (size_t)(N_gu / 2) * 2);
    w->gemm_bytes = gemm;
    w->gemm_counters = gemm_counters;
    w->total = w->gemm + up(gemm);
    return GNF4B_OK;
}

size_t gnf4b_ffn_workspace_bytes(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn,
                                 int32_t max_rows, uint32_t flags) {
    if (ffn_check(fmt, GNF4B_X_BF16, fmt == GNF4B_FMT_NF4 ? GNF4B_S_F32 : GNF4B_S_E8M0, T, G, 1, N_gu, K_gu, N_dn)) return 0;
    DevInfo di;
    if (device_info(&di)) return 0;
    FfnWs w;
    if (ffn_ws_layout(fmt, T, G, N_gu, K_gu, N_dn, max_rows, flags, di, &w)) return 0;
    return w.total;
}

int gnf4b_ffn_grouped(int fmt, int act, const void* x, int x_dtype, int64_t T,
                      const uint8_t* W_gu, int64_t wgu_stride_e, int64_t wgu_stride_n,
                      const void* S_gu, int64_t sgu_stride_e, int64_t sgu_stride_n,
                      const uint8_t* W_dn, int64_t wdn_stride_e, int64_t wdn_stride_n,
                      const void* S_dn, int64_t sdn_stride_e, int64_t sdn_stride_n, int s_dtype,
                      const void* bias_gu, const int32_t* group_offsets, const int32_t* expert_ids, int32_t G, int32_t E,
                      int64_t N_gu, int64_t K_gu, int64_t N_dn, int32_t max_rows, void* out, void* workspace,
                      size_t workspace_bytes, int32_t* status_word, uint32_t flags, void* cuda_stream) {
    int rc = ffn_check(fmt, x_dtype, s_dtype, T, G, E, N_gu, K_gu, N_dn);
    if (rc) return rc;
    if (act != GNF4B_ACT_SILU_GLU && act != GNF4B_ACT_GPT_OSS_GLU) return GNF4B_EINVAL;
    if (T == 0 || G == 0) return GNF4B_OK;
    if (!x || !W_gu || !S_gu || !W_dn || !S_dn || !group_offsets || !expert_ids || !out || !workspace) return GNF4B_EINVAL;
    if (((uintptr_t)x | (uintptr_t)out | (uintptr_t)workspace | (uintptr_t)bias_gu) & 15) return GNF4B_EINVAL;
    DevInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    FfnWs w;
    rc = ffn_ws_layout(fmt, T, G, N_gu, K_gu, N_dn, max_rows, flags, di, &w);
    if (rc) return rc;
    if (workspace_bytes < w.total) return GNF4B_EWORKSPACE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    unsigned char* base = static_cast<unsigned char*>(workspace);
    const int64_t H = N_gu / 2;

    // ---- the fused launch: every group one row, short rows, contiguous 16-byte aligned stacks
    const int elt = (s_dtype == GNF4B_S_F32) ? 4 : (s_dtype == GNF4B_S_BF16 ? 2 : 1);
    const int64_t blk = (fmt == GNF4B_FMT_NF4) ? 64 : 32;
    const int64_t rb[2] = {K_gu / 2, H / 2}, srow[2] = {(K_gu / blk) * elt, (H / blk) * elt};
    auto contiguous = [&](const uint8_t* W, int64_t w_se, int64_t w_sn, const void* S, int64_t s_se, int64_t s_sn, int p) {
        return w_sn == rb[p] && s_sn * elt == srow[p] && (((uintptr_t)W | (uint64_t)w_se) & 15) == 0 &&
               (((uintptr_t)S | (uint64_t)(s_se * elt)) & 15) == 0 && ((8 * srow[p]) & 15) == 0;
    };
    const int au = (int)ceil_div(std::max(K_gu, H), 1024);
    const bool fused = max_rows == 1 && !(flags & GNF4B_FLAG_FFN_UNFUSED) && au <= 3 && (N_gu % 8) == 0 && (N_dn % 8) == 0 &&
                 contiguous(W_gu, wgu_stride_e, wgu_stride_n, S_gu, sgu_stride_e, sgu_stride_n, 0) &&
                 contiguous(W_dn, wdn_stride_e, wdn_stride_n, S_dn, sdn_stride_e, sdn_stride_n, 1) &&
                 (act == GNF4B_ACT_SILU_GLU || fmt == GNF4B_FMT_MXFP4);
    if (fused) {
        FfnArgs fa;
        const int64_t room = (int64_t)di.smem_optin - (int64_t)ffn_smem_bytes(0, 0, (int)H);
        const int64_t per_row = std::max(rb[0] + srow[0], rb[1] + srow[1]);
        // 32 weight rows per stage (two per warp in flight) when three such stages fit the ring, else 16
        int R = 32, rw = 2;
        if (3 * round_up(R * per_row, 128) > room) { R = 16; rw = 1; }
        fa.slot_bytes = (int32_t)round_up(R * per_row, 128);
        fa.stages = (int32_t)std::min<int64_t>(kDMaxStages, room / fa.slot_bytes);
        const int64_t N[2] = {N_gu, N_dn};
        int64_t items_max = 0;
        for (int p = 0; p < 2; ++p) items_max = std::max(items_max, (int64_t)G * ceil_div(N[p], R));
        if (fa.stages >= 3 && items_max < ((int64_t)1 << 31)) {
            const int grid = (int)std::min<int64_t>(di.sm_count, items_max);
            const uint8_t* Wp[2] = {W_gu, W_dn};
            const void* Sp[2] = {S_gu, S_dn};
            const int64_t wse[2] = {wgu_stride_e, wdn_stride_e}, sse[2] = {sgu_stride_e, sdn_stride_e};
            for (int p = 0; p < 2; ++p) {
                FfnPhase& ph = fa.ph[p];
                ph.W = Wp[p]; ph.S = Sp[p]; ph.w_se = wse[p]; ph.s_se = sse[p];
                ph.N = (int32_t)N[p];
                ph.rows_per_stage = R;
                ph.tiles_per_group = (int32_t)ceil_div(N[p], R);
                ph.row_bytes = (int32_t)rb[p];
                ph.scale_row_bytes = (int32_t)srow[p];
                const int64_t items = (int64_t)G * ph.tiles_per_group;
                ph.items_per_cta = (int32_t)(items / grid);
                ph.items_extra = (int32_t)(items % grid);
            }
            fa.x = x; fa.off = group_offsets; fa.eids = expert_ids;
            fa.bias_gu = static_cast<const uint16_t*>(bias_gu);
            fa.gu = reinterpret_cast<uint16_t*>(base + w.gu);
            fa.out = static_cast<uint16_t*>(out);
            fa.counters = reinterpret_cast<int32_t*>(base + w.counters);
            fa.status = status_word;
            fa.T = T; fa.G = G; fa.E = E; fa.K_gu = (int32_t)K_gu; fa.H = (int32_t)H;
            fa.tables_ready = (flags & GNF4B_FLAG_TABLES_READY) ? 1 : 0;
            const size_t smem = ffn_smem_bytes(fa.slot_bytes, fa.stages, (int)H);
            cudaError_t e;
            const bool gpt = act == GNF4B_ACT_GPT_OSS_GLU;
            if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32)
                e = launch_ffn_au<GNF4B_FMT_NF4, GNF4B_S_F32, 0>(fa, au, rw, grid, smem, st);
            else if (fmt == GNF4B_FMT_NF4)
                e = launch_ffn_au<GNF4B_FMT_NF4, GNF4B_S_BF16, 0>(fa, au, rw, grid, smem, st);
            else if (gpt)
                e = launch_ffn_au<GNF4B_FMT_MXFP4, GNF4B_S_E8M0, 1>(fa, au, rw, grid, smem, st);
            else
                e = launch_ffn_au<GNF4B_FMT_MXFP4, GNF4B_S_E8M0, 0>(fa, au, rw, grid, smem, st);
            if (e != cudaSuccess) return cuda_fail(e, "fused FFN launch");
            return GNF4B_OK;
        }
    }

    // ---- three launches, the intermediates in the workspace
    if (bias_gu) return GNF4B_EUNSUPPORTED;          // the bias needs the fused kernel's group walk
    void* gemm_ws = w.gemm_bytes ? base + w.gemm : nullptr;
    rc = gnf4b_gemm_grouped(fmt, GNF4B_OP_FWD, x, x_dtype, T, W_gu, wgu_stride_e, wgu_stride_n, S_gu, s_dtype, sgu_stride_e,
                            sgu_stride_n, group_offsets, expert_ids, G, E, N_gu, K_gu, max_rows, base + w.gu, gemm_ws,
                            w.gemm_bytes, status_word, flags & ~GNF4B_FLAG_FFN_UNFUSED, cuda_stream);
    if (rc) return rc;
    rc = act == GNF4B_ACT_SILU_GLU ? gnf4b_silu_glu(base + w.gu, T, H, base + w.h, cuda_stream)
                                   : gnf4b_glu_gpt_oss(base + w.gu, T, H, nullptr, nullptr, base + w.h, cuda_stream);
    if (rc) return rc;
    return gnf4b_gemm_grouped(fmt, GNF4B_OP_FWD, base + w.h, x_dtype, T, W_dn, wdn_stride_e, wdn_stride_n, S_dn, s_dtype,
                              sdn_stride_e, sdn_stride_n, group_offsets, expert_ids, G, E, N_dn, H, max_rows, out, gemm_ws,
                              w.gemm_bytes, status_word, flags & ~GNF4B_FLAG_FFN_UNFUSED, cuda_stream);
}

static int ffn_staging_layout(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn, uint32_t flags,
                              const DevInfo& di, FfnStaging* f) {
    auto up = [](size_t v) { return (size_t)round_up((int64_t)v, 256); };
    size_t worst = 0;
    for (int32_t mr : {1, -1}) {
        FfnWs w;
        const int rc = ffn_ws_layout(fmt, T, G, N_gu, K_gu, N_dn, mr, flags, di, &w);
        if (rc) return rc;
        worst = std::max(worst, w.total);
    }
    f->ws_bytes = worst;
    f->tab_bytes = (size_t)(2 * (int64_t)G + 2) * 4;
    f->x_bytes = (size_t)T * (size_t)K_gu * 2;
    f->out_bytes = (size_t)T * (size_t)N_dn * 2;
    f->tab = up(f->ws_bytes);
    f->x = f->tab + up(f->tab_bytes);
    f->out = f->x + up(f->x_bytes);
    f->total = f->out + up(f->out_bytes);
    return GNF4B_OK;
}

size_t gnf4b_ffn_host_staging_bytes(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn,
                                    uint32_t flags) {
    if (ffn_check(fmt, GNF4B_X_BF16, fmt == GNF4B_FMT_NF4 ? GNF4B_S_F32 : GNF4B_S_E8M0, T, G, 1, N_gu, K_gu, N_dn)) return 0;
    DevInfo di;
    if (device_info(&di)) return 0;
    FfnStaging f;
    if (ffn_staging_layout(fmt, T, G, N_gu, K_gu, N_dn, flags, di, &f)) return 0;
    return f.total;
}

int gnf4b_ffn_grouped_host(int fmt, const void* x_host, int x_dtype, int64_t T,
                           const uint8_t* W_gu, int64_t wgu_stride_e, int64_t wgu_stride_n,
                           const void* S_gu, int64_t sgu_stride_e, int64_t sgu_stride_n,
                           const uint8_t* W_dn, int64_t wdn_stride_e, int64_t wdn_stride_n,
                           const void* S_dn, int64_t sdn_stride_e, int64_t sdn_stride_n, int s_dtype,
                           const int32_t* sizes_host, const int32_t* expert_ids_host, int32_t G, int32_t E,
                           int64_t N_gu, int64_t K_gu, int64_t N_dn, void* out_host, void* staging,
                           size_t staging_bytes, int32_t* status_host, uint32_t flags, void* cuda_stream) {
    int rc = ffn_check(fmt, x_dtype, s_dtype, T, G, E, N_gu, K_gu, N_dn);
    if (rc) return rc;
    if (status_host) *status_host = 0;
    if (G > 0 && (!sizes_host || !expert_ids_host)) return GNF4B_EINVAL;
    int64_t total = 0;
    int32_t max_rows = 0;
    for (int32_t g = 0; g < G; ++g) {
        const int32_t n = sizes_host[g], e = expert_ids_host[g];
        if (n < 0 || (e != GNF4B_PAD_EXPERT && (e < 0 || e >= E))) return GNF4B_EINVAL;
        total += n;
        max_rows = std::max(max_rows, n);
    }
    if (total != T) return GNF4B_EINVAL;
    if (T == 0 || G == 0) return GNF4B_OK;
    if (!x_host || !out_host || !staging || ((uintptr_t)staging & 255)) return GNF4B_EINVAL;
    DevInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    FfnStaging f;
    rc = ffn_staging_layout(fmt, T, G, N_gu, K_gu, N_dn, flags, di, &f);
    if (rc) return rc;
    if (staging_bytes < f.total) return GNF4B_EWORKSPACE;
    FfnWs w;
    rc = ffn_ws_layout(fmt, T, G, N_gu, K_gu, N_dn, max_rows, flags, di, &w);
    if (rc) return rc;

    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    unsigned char* base = static_cast<unsigned char*>(staging);
    int32_t* d_off = reinterpret_cast<int32_t*>(base + f.tab);
    int32_t* d_ids = d_off + (G + 1);
    int32_t* d_status = d_ids + G;
    cudaError_t e;

    PinnedBlock& pin = thread_pinned_block();
    e = ensure_pinned_block(pin);
    if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc(pinned block)");
    const size_t tab_span = f.x - f.tab;
    const bool tab_fits = tab_span <= kHostPinnedBytes;
    const bool x_rides = tab_fits && tab_span + f.x_bytes <= kHostPinnedBytes;
    const bool direct = x_rides && pin.dev && f.out_bytes <= kHostPinnedBytes && f.out_bytes % 16 == 0 &&
                        w.gu % 16 == 0 && w.gemm_counters % 16 == 0 && !(flags & GNF4B_FLAG_HOST_COPIES);
    std::vector<int32_t> big_tab;
    int32_t* t = tab_fits ? reinterpret_cast<int32_t*>(pin.p) : (big_tab.resize(2 * (size_t)G + 2), big_tab.data());
    t[0] = 0;
    for (int32_t g = 0; g < G; ++g) t[g + 1] = t[g] + sizes_host[g];
    std::memcpy(t + G + 1, expert_ids_host, (size_t)G * 4);
    t[2 * (size_t)G + 1] = 0;
    if (direct) {
        // small call: in and out through the pinned block by two small kernels instead of the copy engines; the
        // counters that must start at zero are cleared by the first of them
        std::memcpy(pin.p + tab_span, x_host, f.x_bytes);
        e = host_stage_in(pin, d_off, tab_span + f.x_bytes, base, w.gu, w.gemm_counters ? base + w.gemm : nullptr,
                          w.gemm_counters, st);
        if (e != cudaSuccess) return cuda_fail(e, "host_stage_in launch");
        rc = gnf4b_ffn_grouped(fmt, GNF4B_ACT_SILU_GLU, base + f.x, x_dtype, T, W_gu, wgu_stride_e, wgu_stride_n, S_gu,
                               sgu_stride_e, sgu_stride_n, W_dn, wdn_stride_e, wdn_stride_n, S_dn, sdn_stride_e, sdn_stride_n,
                               s_dtype, nullptr, d_off, d_ids, G, E, N_gu, K_gu, N_dn, max_rows, base + f.out, base, w.total,
                               d_status, flags & ~GNF4B_FLAG_TABLES_READY, cuda_stream);
        if (rc) { cudaStreamSynchronize(st); return rc; }
        return host_stage_out_wait(pin, base + f.out, f.out_bytes, d_status, out_host, status_host, st);
    }
    if (x_rides) {
        std::memcpy(pin.p + tab_span, x_host, f.x_bytes);
        e = cudaMemcpyAsync(d_off, pin.p, tab_span + f.x_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(tables + x)");
    } else {
        e = cudaMemcpyAsync(d_off, t, f.tab_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(tables)");
        e = cudaMemcpyAsync(base + f.x, x_host, f.x_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(x)");
    }
    auto fail = [&](int code) { cudaStreamSynchronize(st); return code; };   // queued copies read host memory
    // what must start at zero: the group counters of the fused launch and the arrival counters of split-K GEMMs
    e = cudaMemsetAsync(base, 0, w.gu, st);
    if (e == cudaSuccess && w.gemm_counters) e = cudaMemsetAsync(base + w.gemm, 0, w.gemm_counters, st);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemsetAsync(counters)"));
    // the tables were uploaded by the copy above: ready when the kernels start
    rc = gnf4b_ffn_grouped(fmt, GNF4B_ACT_SILU_GLU, base + f.x, x_dtype, T, W_gu, wgu_stride_e, wgu_stride_n, S_gu,
                           sgu_stride_e, sgu_stride_n, W_dn, wdn_stride_e, wdn_stride_n, S_dn, sdn_stride_e, sdn_stride_n,
                           s_dtype, nullptr, d_off, d_ids, G, E, N_gu, K_gu, N_dn, max_rows, base + f.out, base, w.total,
                           d_status, flags | GNF4B_FLAG_TABLES_READY, cuda_stream);
    if (rc) return fail(rc);
    e = cudaMemcpyAsync(out_host, base + f.out, f.out_bytes, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemcpyAsync(out)"));
    if (status_host) {
        e = cudaMemcpyAsync(status_host, d_status, 4, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemcpyAsync(status)"));
    }
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return GNF4B_OK;
}

int gnf4b_combine_rows(const void* rows, int64_t P, const int64_t* pos, const float* weights, int32_t k, int64_t M,
                       int64_t H, void* out, int32_t* status_word, void* cuda_stream) {
    if (P < 0 || M < 0 || H <= 0 || k <= 0) return GNF4B_EINVAL;
    if (M > 0 && (!pos || !weights || !out || (P > 0 && !rows))) return GNF4B_EINVAL;
    if (M == 0) return GNF4B_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    const bool vec = (H % 8) == 0 && ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int64_t work = M * (vec ? H / 8 : H);
    const int grid = (int)std::min<int64_t>(ceil_div(work, 256), 148 * 16);
    if (vec)
        combine_rows_kernel<8><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(rows), pos, weights, k, M, H, P,
                                                     static_cast<uint16_t*>(out), status_word);
    else
        combine_rows_kernel<1><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(rows), pos, weights, k, M, H, P,
                                                     static_cast<uint16_t*>(out), status_word);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "combine_rows launch");
}

int gnf4b_route_topk(const float* logits, int64_t T, int32_t E, int32_t k, int32_t mode, int32_t norm, int64_t* idx,
                     float* weights, void* cuda_stream) {
    if (T < 0 || E <= 0 || k < 1 || k > E || k > 32 || (mode != 0 && mode != 1)) return GNF4B_EINVAL;
    if (T > 0 && (!logits || !idx || !weights)) return GNF4B_EINVAL;
    if (T == 0) return GNF4B_OK;
    const int warps = 4;
    route_topk_kernel<<<(unsigned)ceil_div(T, warps), warps * 32, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
        logits, T, E, k, mode, norm, idx, weights);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "route_topk launch");
}

int gnf4b_ep_plan(const int64_t* idx, int32_t P, int32_t k, int32_t n_experts, int32_t e_local, int32_t cap,
                  const void* hidden, int64_t H, int32_t* counts, int64_t* slot, void* send, int32_t* status_word,
                  void* cuda_stream) {
    if (P < 0 || k <= 0 || n_experts <= 0 || e_local <= 0 || n_experts % e_local || cap < 0 || H <= 0) return GNF4B_EINVAL;
    if (P > kEpPlanMax || n_experts > kEpPlanMax) return GNF4B_ETOOBIG;
    if (!counts || (P > 0 && (!idx || !hidden || !slot || !send))) return GNF4B_EINVAL;
    ep_plan_kernel<<<1, kEpPlanThreads, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
        idx, P, k, n_experts, e_local, cap, static_cast<const uint16_t*>(hidden), H, counts, slot,
        static_cast<uint16_t*>(send), status_word);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_plan launch");
}

int gnf4b_ep_push_blocks(int32_t n, const void* const* src, void* const* dst, const int64_t* bytes, int32_t* const* flags,
                         int32_t step, int32_t first_block, int32_t* done_counter, void* cuda_stream) {
    if (n < 0 || n > kEpPeerMaxWorld || !done_counter) return GNF4B_EINVAL;
    if (n == 0) return GNF4B_OK;
    if (!src || !dst || !bytes) return GNF4B_EINVAL;
    EpPushArgs a;
    std::memset(&a, 0, sizeof(a));
    int64_t chunks = 0;
    for (int b = 0; b < n; ++b) {
        if (bytes[b] < 0 || (bytes[b] % 16)) return GNF4B_ESHAPE;
        if (bytes[b] > 0 && (!src[b] || !dst[b] || ((reinterpret_cast<uintptr_t>(src[b]) | reinterpret_cast<uintptr_t>(dst[b])) & 15)))
            return GNF4B_EINVAL;
        a.src[b] = static_cast<const uint8_t*>(src[b]);
        a.dst[b] = static_cast<uint8_t*>(dst[b]);
        a.bytes[b] = bytes[b];
        a.flag[b] = flags ? flags[b] : nullptr;
        chunks += ceil_div(bytes[b], kEpPushChunk);
    }
    a.n = n;
    a.step = step;
    a.rot = ((first_block % n) + n) % n;
    a.done_counter = done_counter;
    DevInfo di;
    int rc = device_info(&di);
    if (rc) return rc;
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(chunks, 2 * (int64_t)di.sm_count));
    ep_push_blocks_kernel<<<grid, kEpPeerThreads, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(a);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_push_blocks launch");
}

int gnf4b_ep_wait_flags(const int32_t* flags, int32_t world, int32_t step, int32_t timeout_ms, int32_t* status_word,
                        void* cuda_stream) {
    if (!flags || world <= 0 || world > kEpPeerMaxWorld || timeout_ms <= 0) return GNF4B_EINVAL;
    ep_wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(flags, world, step,
                                                                                   (uint64_t)timeout_ms * 1000000ull, status_word);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_wait_flags launch");
}

size_t gnf4b_ep_plan_large_scratch_bytes(int64_t P, int32_t n_experts) {
    if (P <= 0 || n_experts <= 0 || n_experts > 1024) return 0;
    return (size_t)ceil_div(P, (int64_t)kEpChunk) * (size_t)(2 * n_experts + 1) * 4;
}

int gnf4b_ep_plan_large(const int64_t* idx, int64_t P, int32_t k, int32_t n_experts, int32_t e_local, int32_t cut,
                        const void* hidden, int64_t H, int32_t* counts, int64_t* pos, void* send, void* scratch,
                        size_t scratch_bytes, int32_t* status_word, void* cuda_stream) {
    if (P < 0 || k <= 0 || n_experts <= 0 || e_local <= 0 || n_experts % e_local || cut < 0 || cut > e_local || H <= 0)
        return GNF4B_EINVAL;
    if (n_experts > 1024 || P > ((int64_t)1 << 26)) return GNF4B_ETOOBIG;
    if (H % 8) return GNF4B_ESHAPE;
    if (!counts || (P > 0 && (!idx || !hidden || !pos || !send))) return GNF4B_EINVAL;
    if ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(send)) & 15) return GNF4B_EINVAL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    if (P == 0) {
        cudaError_t e0 = cudaMemsetAsync(counts, 0, (size_t)n_experts * 4, st);
        return e0 == cudaSuccess ? GNF4B_OK : cuda_fail(e0, "cudaMemsetAsync(counts)");
    }
    if (!scratch || scratch_bytes < gnf4b_ep_plan_large_scratch_bytes(P, n_experts)) return GNF4B_EWORKSPACE;
    int32_t* hist = static_cast<int32_t*>(scratch);
    const int n_ctas = (int)ceil_div(P, (int64_t)kEpChunk);
    ep_large_hist_kernel<<<n_ctas, kEpLargeThreads, 0, st>>>(idx, P, n_experts, e_local, cut, hist, status_word);
    ep_large_starts_kernel<<<1, 1024, 0, st>>>(hist, n_ctas, n_experts, counts);
    ep_large_place_kernel<<<n_ctas, kEpLargeThreads, 0, st>>>(idx, P, n_experts, e_local, cut, hist, pos);
    const int64_t items = P * (H / 8);
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(items, (int64_t)kEpLargeThreads), 148 * 32);
    ep_large_rows_kernel<<<grid, kEpLargeThreads, 0, st>>>(static_cast<const uint16_t*>(hidden), P, k, H, pos,
                                                          static_cast<uint16_t*>(send));
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_plan_large launch");
}

int gnf4b_ep_offsets(const int32_t* recv_counts, int32_t world, int32_t e_local, int32_t cap, int32_t* offsets,
                     int32_t* status_word, void* cuda_stream) {
    if (world <= 0 || e_local <= 0 || cap < 0 || !recv_counts || !offsets) return GNF4B_EINVAL;
    if ((int64_t)world * e_local > kEpPlanMax) return GNF4B_ETOOBIG;
    ep_offsets_kernel<<<1, kEpOffsetsThreads, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(recv_counts, world, e_local, cap, offsets,
                                                                              status_word);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_offsets launch");
}

static_assert(sizeof(gnf4b_ep_peer_ctx) == sizeof(EpPeerCtx) && GNF4B_EP_MAX_WORLD == kEpPeerMaxWorld,
              "the public exchange context and the kernels' argument struct are the same bytes");

static int ep_peer_ctx(const gnf4b_ep_peer_ctx* c, int32_t cap, EpPeerCtx* out) {
    if (!c || c->world <= 0 || c->world > kEpPeerMaxWorld || c->rank < 0 || c->rank >= c->world || c->e_local <= 0 ||
        c->cap_max <= 0 || c->H <= 0 || (c->H % 8) || cap < 0)
        return GNF4B_EINVAL;
    if (cap > c->cap_max || (int64_t)c->world * c->e_local > kEpPlanMax || (int64_t)c->world * cap > kEpPlanMax)
        return GNF4B_ETOOBIG;
    for (int r = 0; r < c->world; ++r)
        if (!c->peers[r] || (reinterpret_cast<uintptr_t>(c->peers[r]) & 255)) return GNF4B_EINVAL;
    std::memcpy(out, c, sizeof(EpPeerCtx));
    return GNF4B_OK;
}

int gnf4b_ep_peer_layout(int32_t world, int32_t e_local, int32_t cap_max, int64_t H, int64_t* out3) {
    if (world <= 0 || world > kEpPeerMaxWorld || e_local <= 0 || cap_max <= 0 || H <= 0 || (H % 8) || !out3) return GNF4B_EINVAL;
    const EpPeerLayout L = ep_peer_layout(world, e_local, cap_max, H);
    out3[0] = L.total;
    out3[1] = L.recv_rows;
    out3[2] = L.ret_ll;
    return GNF4B_OK;
}

int gnf4b_ep_peer_dispatch(const gnf4b_ep_peer_ctx* ctx, const int64_t* idx, int32_t P, int32_t k, int32_t n_experts,
                           int32_t cap, const void* hidden, int64_t* slot, int32_t one_row_groups, int32_t* offsets,
                           int32_t* expert_ids, int32_t* status_word, void* cuda_stream) {
    EpPeerCtx cx;
    int rc = ep_peer_ctx(ctx, cap, &cx);
    if (rc) return rc;
    if (P < 0 || k <= 0 || n_experts != cx.world * cx.e_local) return GNF4B_EINVAL;
    if (P > kEpPlanMax || n_experts > kEpPlanMax) return GNF4B_ETOOBIG;
    if (P > 0 && (!idx || !hidden || !slot)) return GNF4B_EINVAL;
    if (!offsets || (one_row_groups && !expert_ids)) return GNF4B_EINVAL;
    if (reinterpret_cast<uintptr_t>(hidden) & 15) return GNF4B_EINVAL;
    const int32_t n_groups = one_row_groups ? cx.world * cap : cx.e_local;
    // one pass of 16 bytes per thread where that needs no more than 32 CTAs (each repeats the small plan); about cap
    // of the world * cap row slots are in use on the receiving side
    const int64_t rows = std::max<int64_t>(P, cap);
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(32, ceil_div(rows * cx.H * 2, (int64_t)4096)));
    cudaError_t e = launch_pdl(ep_peer_dispatch_kernel, grid, kEpPeerThreads, reinterpret_cast<cudaStream_t>(cuda_stream), cx,
                               idx, P, k, n_experts, cap, static_cast<const uint16_t*>(hidden), slot, one_row_groups ? 1 : 0,
                               n_groups, offsets, expert_ids, status_word);
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_peer_dispatch launch");
}

int gnf4b_ep_peer_combine(const gnf4b_ep_peer_ctx* ctx, int32_t cap, const void* y, const int64_t* slot, const float* weights,
                          int32_t k, int64_t M, void* out, int32_t* status_word, void* cuda_stream) {
    EpPeerCtx cx;
    int rc = ep_peer_ctx(ctx, cap, &cx);
    if (rc) return rc;
    if (!y || k <= 0 || M < 0 || (M > 0 && (!slot || !weights || !out))) return GNF4B_EINVAL;
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(y)) & 15) return GNF4B_EINVAL;
    const int64_t rows = std::max<int64_t>(M, cap);
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(32, ceil_div(rows * cx.H * 2, (int64_t)4096)));
    cudaError_t e = launch_pdl(ep_peer_combine_kernel, grid, kEpPeerThreads, reinterpret_cast<cudaStream_t>(cuda_stream), cx, cap,
                               static_cast<const uint16_t*>(y), slot, weights, k, M, static_cast<uint16_t*>(out), status_word);
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "ep_peer_combine launch");
}

int gnf4b_gather_rows_by_id(void* dst, int64_t row_bytes, int32_t n_slots, const void* src, int32_t n_rows_src,
                            const int32_t* ids, const int32_t* have_ids, int32_t* status_word, void* cuda_stream) {
    if (row_bytes <= 0 || n_slots < 0 || n_rows_src < 0) return GNF4B_EINVAL;
    if (row_bytes % 8) return GNF4B_ESHAPE;
    if (n_slots == 0) return GNF4B_OK;
    if (!dst || !src || !ids || ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 7)) return GNF4B_EINVAL;
    if (n_slots > 65535) return GNF4B_ETOOBIG;
    const dim3 grid((unsigned)ceil_div(row_bytes, kGatherChunk), (unsigned)n_slots);
    gather_rows_kernel<0><<<grid, kGatherThreads, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<uint8_t*>(dst), row_bytes, static_cast<const uint8_t*>(src), ids, have_ids, nullptr, nullptr, n_rows_src,
        status_word);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "gather_rows_by_id launch");
}

int gnf4b_gather_rows_addr(void* dst, int64_t row_bytes, int32_t n_slots, const int64_t* want_addr, const int64_t* have_addr,
                           const int64_t* pieces, int32_t n_pieces, int64_t max_piece_bytes, void* cuda_stream) {
    if (row_bytes <= 0 || n_slots < 0 || n_pieces < 0) return GNF4B_EINVAL;
    if (row_bytes % 8 || max_piece_bytes % 8) return GNF4B_ESHAPE;
    if (n_slots == 0) return GNF4B_OK;
    if (!dst || !want_addr || (reinterpret_cast<uintptr_t>(dst) & 7)) return GNF4B_EINVAL;
    if (n_slots > 65535 || n_pieces > 65535) return GNF4B_ETOOBIG;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    if (n_pieces == 0) {
        const dim3 grid((unsigned)ceil_div(row_bytes, kGatherChunk), (unsigned)n_slots);
        gather_rows_kernel<1><<<grid, kGatherThreads, 0, st>>>(static_cast<uint8_t*>(dst), row_bytes, nullptr, nullptr, nullptr,
                                                              want_addr, have_addr, 0, nullptr);
    } else {
        if (!pieces || max_piece_bytes <= 0 || max_piece_bytes > row_bytes) return GNF4B_EINVAL;
        const dim3 grid((unsigned)ceil_div(max_piece_bytes, kGatherChunk), (unsigned)n_pieces, (unsigned)n_slots);
        gather_rows_pieces_kernel<<<grid, kGatherThreads, 0, st>>>(static_cast<uint8_t*>(dst), row_bytes, want_addr, have_addr,
                                                                   pieces);
    }
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? GNF4B_OK : cuda_fail(e, "gather_rows_addr launch");
}

int gnf4b_dequant(int fmt, const uint8_t* W, int64_t w_stride_e, int64_t w_stride_n, const void* S,
                  int s_dtype, int64_t s_stride_e, int64_t s_stride_n, int32_t E, int64_t N, int64_t K,
                  float* out_f32, void* cuda_stream) {
    int rc = check_shape(fmt, GNF4B_OP_FWD, GNF4B_X_BF16, s_dtype, 0, 0, E, N, K);
    if (rc) return rc;
    if (!W || !S || !out_f32) return GNF4B_EINVAL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    const int64_t total = (int64_t)E * N * (K / 2);
    const int grid = (int)std::min<int64_t>(ceil_div(total, 256), 148 * 16);
    if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32)
        dequant_kernel<GNF4B_FMT_NF4, GNF4B_S_F32><<<grid, 256, 0, st>>>(W, w_stride_e, w_stride_n, S, s_stride_e, s_stride_n, E, N, K, out_f32);
    else if (fmt == GNF4B_FMT_NF4)
        dequant_kernel<GNF4B_FMT_NF4, GNF4B_S_BF16><<<grid, 256, 0, st>>>(W, w_stride_e, w_stride_n, S, s_stride_e, s_stride_n, E, N, K, out_f32);
    else
        dequant_kernel<GNF4B_FMT_MXFP4, GNF4B_S_E8M0><<<grid, 256, 0, st>>>(W, w_stride_e, w_stride_n, S, s_stride_e, s_stride_n, E, N, K, out_f32);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "dequant kernel launch");
    return GNF4B_OK;
}

}  // extern "C"

#ifdef GNF4B_EP_TRACE
extern "C" int gnf4b_ep_trace_read(unsigned long long* host, int max_events) {
    unsigned int n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, gnf4b::g_ep_trace_n, sizeof(n));
    if ((int)n > max_events) n = max_events;
    if (n > 4096) n = 4096;
    cudaMemcpyFromSymbol(host, gnf4b::g_ep_trace, (size_t)n * 16);
    unsigned int z = 0;
    cudaMemcpyToSymbol(gnf4b::g_ep_trace_n, &z, sizeof(z));
    return (int)n;
}
#endif
