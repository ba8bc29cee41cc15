// Exact search that allocates nothing.
//
// Some callers are not allowed to allocate device memory at the moment they search: a serving
// process that handed all of HBM to its own pool at start-up (cudaMalloc would fail or fragment
// that pool), or a latency-critical loop that cannot afford the device-wide synchronisation that
// cudaMalloc / cudaFree imply.  The regular search path grows its scratch buffers with cudaMalloc
// on first use; this entry point instead runs the same kernels (query preparation, distance GEMM
// with the append epilogue writing every key, fp32 refinement, exact top-k selection, result
// emission) with all scratch carved out of one file-scope __device__ array of fixed size.
//
// Limits: a Flat or Int8Flat index; n * round_up(ntotal, 256) <= kMaxCandidates keys;
// k <= kMaxK.  Larger requests are rejected with B200IDX_ERR_INVALID_PARAM.
//
// The array is shared by every call in the process (per GPU): it keeps the previous call's
// contents, so everything that must start clean is re-initialised on every call, and two calls
// that overlap on the same GPU race on it.  The first call on a device looks up the array's
// device address (cudaGetSymbolAddress); make that first call before any stream capture begins.
#include "../../include/b200idx.h"

#include <mutex>
#include <stdexcept>
#include <string>

#include "c_api_internal.h"
#include "dist_gemm.cuh"
#include "flat_index.h"
#include "select.cuh"

using namespace b200;

namespace {

constexpr size_t kMaxCandidates = size_t(1) << 20;   // n * padded ntotal
constexpr int kMaxKNoAlloc = 1024;
constexpr int kMaxQueries = 1024;
constexpr size_t kMaxQueryElems = size_t(1) << 19;                // n * d
constexpr size_t kCandBytes = kMaxCandidates * 8;                 // 8 MiB of (key, position) pairs
constexpr size_t kSelBudget = size_t(1) << 20;                    // n * k <= 128 Ki selected pairs (1 MiB)
constexpr size_t kQopBytes = (size_t(1) << 20) + (size_t(32) << 10);   // n * d * 2 <= 1 MiB operand copy + 16 folded columns per row
constexpr size_t kSmallBytes = size_t(64) << 10;                  // norms, slack, thresholds, flags
constexpr size_t kArenaBytes = kCandBytes + kSelBudget + kQopBytes + kSmallBytes;  // 10 MiB + 96 KiB

// Host code must not use this name as an address: it is a host-side stand-in.  The device
// address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_arena[kArenaBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_arena_ptr[kMaxDevices] = {};
std::mutex g_arena_mutex;

unsigned char* arena_for_device(int device) {
    if (device < 0 || device >= kMaxDevices) throw std::invalid_argument("device ordinal out of range");
    std::lock_guard<std::mutex> l(g_arena_mutex);
    if (!g_arena_ptr[device]) {
        // once per device, with that device current
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_arena);
        if (e != cudaSuccess || !p)
            throw std::runtime_error(std::string("cudaGetSymbolAddress(scratch arena): ") + cudaGetErrorString(e));
        g_arena_ptr[device] = static_cast<unsigned char*>(p);
    }
    return g_arena_ptr[device];
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" int b200idx_search_device_noalloc(b200idx_t* h, int64_t n, const void* x_dev, int k, float* D_dev,
                                             int64_t* I_dev) {
    if (!h) return B200IDX_ERR_INVALID_PARAM;
    return b200_capi::guarded(h, [&] {
        FlatIndex* ix = b200_capi::flat_of(h);
        if (!ix) throw std::invalid_argument("the no-allocation search applies to Flat and Int8Flat indexes");
        if (n <= 0 || !x_dev || !D_dev || !I_dev) throw std::invalid_argument("n must be > 0, pointers non-NULL");
        if (k <= 0 || k > kMaxKNoAlloc) throw std::invalid_argument("k must be in [1, 1024] for the no-allocation search");
        const FlatIndex::RawView v = ix->raw_view();
        if (v.n <= 0) throw std::invalid_argument("the no-allocation search needs a non-empty index");
        const int d = ix->d();
        const int64_t n_pad = (v.n + kTileB - 1) / kTileB * kTileB;
        if (n > kMaxQueries || static_cast<size_t>(n) * static_cast<size_t>(n_pad) > kMaxCandidates)
            throw std::invalid_argument("request exceeds the static scratch: n * round_up(ntotal, 256) must be <= 2^20");
        // The operand copy of an fp32 index is op_cols() = d + 16 bf16 values wide (the folded columns), so
        // n * d <= 2^19 together with n <= 1024 keeps n * op_cols() * 2 within kQopBytes.
        if (static_cast<size_t>(n) * k * 8 > kSelBudget || static_cast<size_t>(n) * d > kMaxQueryElems ||
            static_cast<size_t>(n) * ix->op_cols() * 2 > kQopBytes)
            throw std::invalid_argument("request exceeds the static scratch: n * k <= 131072 and n * d <= 524288");

        DeviceGuard g(ix->device());
        unsigned char* arena = arena_for_device(ix->device());
        cudaStream_t st = ix->stream();
        const int nq = static_cast<int>(n);
        const int dtype = ix->dtype();
        const bool is_int = dtype == kI8;
        const uint32_t cap = static_cast<uint32_t>(n_pad);

        // carve the arena
        size_t off = 0;
        uint64_t* cand = reinterpret_cast<uint64_t*>(arena + off);
        off += kCandBytes;
        uint64_t* sel = reinterpret_cast<uint64_t*>(arena + off);
        off += kSelBudget;
        void* qop = arena + off;
        off += kQopBytes;
        unsigned char* small = arena + off;
        void* qnorm = small;
        float* eps = reinterpret_cast<float*>(small + align_up(size_t(nq) * 4, 256));
        uint32_t* tau = reinterpret_cast<uint32_t*>(small + 2 * align_up(size_t(nq) * 4, 256));
        int* err = reinterpret_cast<int*>(small + 3 * align_up(size_t(nq) * 4, 256));

        // everything the kernels read before writing starts clean on every call
        B200_CUDA_CHECK(cudaMemsetAsync(cand, 0xFF, static_cast<size_t>(nq) * cap * 8, st));
        B200_CUDA_CHECK(cudaMemsetAsync(err, 0, sizeof(int), st));
        B200_CUDA_CHECK(launch_fill_u32(tau, nq, is_int ? 0xFFFFFFFFu : 0xFF800000u, st));

        const void* xq_op = x_dev;
        if (dtype == kF32) {
            B200_CUDA_CHECK(launch_prep_queries_f32(static_cast<const float*>(x_dev), nq, d, ix->metric(), v.max_norm,
                                                    qop, static_cast<float*>(qnorm), eps, st));
            xq_op = qop;
        } else if (dtype == kF16) {
            // fp16 index: queries arrive as float, the operand copy lives in the arena
            B200_CUDA_CHECK(launch_f32_to_f16(static_cast<const float*>(x_dev), static_cast<int64_t>(nq) * d, qop, st));
            B200_CUDA_CHECK(launch_prep_queries_f16(qop, nq, d, static_cast<float*>(qnorm), st));
            xq_op = qop;
        } else {
            B200_CUDA_CHECK(launch_prep_queries_i8(static_cast<const int8_t*>(x_dev), nq, d,
                                                   static_cast<int32_t*>(qnorm), st));
        }

        const int kind = ix->gemm_kind_public();
        CUtensorMap map_a, map_b;
        if (!v.use_simt) {
            if (encode_operand_map(&map_b, kind, v.operand, v.n, ix->op_cols(), kTileB) != 0 ||
                encode_operand_map(&map_a, kind, xq_op, nq, ix->op_cols(), kTileQ) != 0)
                throw std::runtime_error("cuTensorMapEncodeTiled failed");
        }
        GemmArgs a{};
        a.A = xq_op;
        a.B = v.operand;
        a.d = ix->op_cols();
        a.nq = nq;
        a.N = v.n;
        a.n_tiles_total = static_cast<int>(n_pad / kTileB);
        a.n_tiles_sel = a.n_tiles_total;
        a.tile_first = 0;
        a.metric = ix->metric();
        a.bnorm = v.norms;
        a.qnorm_i32 = ix->dtype() == kI8 ? static_cast<const int32_t*>(qnorm) : nullptr;
        a.tau = tau;
        a.cand = cand;
        a.counts = nullptr;
        a.cap = cap;
        a.direct = 1;
        a.err = err;
        a.prof = nullptr;
        GemmLaunch L{};
        L.kind = kind;
        L.mode = kModeAppend;
        L.burst = 32;
        L.simt = v.use_simt ? 1 : 0;
        L.num_sms = v.num_sms;
        B200_CUDA_CHECK(launch_dist_gemm(L, a, &map_a, &map_b, st));
        if (dtype == kF32)
            B200_CUDA_CHECK(launch_refine_f32(cand, nullptr, static_cast<uint32_t>(v.n), cap, nq, d, ix->metric(),
                                              static_cast<const float*>(x_dev), v.rows_f32, st));
        B200_CUDA_CHECK(launch_select_topk(cand, nullptr, static_cast<uint32_t>(v.n), cap, nq, k, sel, nullptr, st));
        EmitArgs e{};
        e.sel = sel;
        e.nq = nq;
        e.k = k;
        e.metric = ix->metric();
        e.mode = is_int ? 2 : (dtype == kF32 ? 1 : 0);
        e.qnorm = qnorm;
        e.labels = v.labels;
        e.D = D_dev;
        e.I = I_dev;
        e.ldk = k;
        e.qmap = nullptr;
        B200_CUDA_CHECK(launch_emit(e, st));
        int herr = 0;
        B200_CUDA_CHECK(cudaMemcpyAsync(&herr, err, sizeof(int), cudaMemcpyDeviceToHost, st));
        B200_CUDA_CHECK(cudaStreamSynchronize(st));
        if (herr) throw std::runtime_error("device pipeline reported an error word (bounded wait ran out)");
    });
}
