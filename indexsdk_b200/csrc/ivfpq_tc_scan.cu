// List-major IVFPQ filter scan on tcgen05 (see ivfpq_tc_scan.cuh for the arithmetic).
#include "ivfpq_tc_scan.cuh"

#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr uint32_t kNoPosTc = 0xFFFFFFFFu;
constexpr float kPosInf = __builtin_huge_valf();

// ---------------------------------------------------------------------------------------
// preparation kernels
// ---------------------------------------------------------------------------------------
__global__ void tc_keys_kernel(const int64_t* cI, int64_t npairs, int nlist, int32_t* keys, int32_t* vals) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int64_t l = cI[i];
    keys[i] = (l >= 0 && l < nlist) ? static_cast<int32_t>(l) : nlist;
    vals[i] = static_cast<int32_t>(i);
}

__global__ void tc_bounds_kernel(const int32_t* keys, int64_t npairs, int nlist, int32_t* first, int32_t* last) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int32_t k = keys[i];
    if (k >= nlist) return;
    if (i == 0 || keys[i - 1] != k) first[k] = static_cast<int32_t>(i);
    if (i + 1 == npairs || keys[i + 1] != k) last[k] = static_cast<int32_t>(i + 1);
}

// The 16 code bytes of a slot are stored rotated by (slot mod 16): canonical[m] = stored[(m - rot) & 15].
// Returns the canonical bytes as four little-endian words (a 128-bit rotate left by rot bytes).
__device__ __forceinline__ uint4 unrotate_code(uint4 cw, uint32_t rot) {
    uint32_t w0 = cw.x, w1 = cw.y, w2 = cw.z, w3 = cw.w;
    if (rot & 4u) { const uint32_t tmp = w3; w3 = w2; w2 = w1; w1 = w0; w0 = tmp; }
    if (rot & 8u) { uint32_t tmp = w0; w0 = w2; w2 = tmp; tmp = w1; w1 = w3; w3 = tmp; }
    const uint32_t sh = (rot & 3u) * 8u;
    return make_uint4(__funnelshift_l(w3, w0, sh), __funnelshift_l(w0, w1, sh), __funnelshift_l(w1, w2, sh),
                      __funnelshift_l(w2, w3, sh));
}

// error bound of the fp16 product for a pair whose coarse distance is cd, times the factor 2 with
// which the accumulator enters the distance
__device__ __forceinline__ float pair_err(float cd, float cb_bound) {
    const float rc = sqrtf(fmaxf(cd, 0.f));
    return 2.02f * (kTcErrRel * rc * cb_bound + kTcErrAbs * (rc + cb_bound));
}

__device__ __forceinline__ uint32_t order_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unorder_bits(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o);
}

// One warp per query: distances (fp32 arithmetic on the fp16 codewords, plus the pair's error
// bound: upper bounds of what the scan produces) to the codes of the nearest list -- and of the
// second nearest when the first holds fewer than 128 -- at most 1024 of them; tau is the k'-th
// smallest, plus fp32 rounding slack.
constexpr int kHeadWarps = 8, kHeadMax = 1024;
__global__ void __launch_bounds__(kHeadWarps * 32)
tc_head_tau_kernel(const TcScanArgs a, const int64_t* cI, float err_rel, float t2_bound, float* tau) {
    __shared__ float s_x[kHeadWarps][2][kTcDim];
    __shared__ uint32_t s_v[kHeadWarps][kHeadMax];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t q = static_cast<int64_t>(blockIdx.x) * kHeadWarps + warp;
    if (q >= a.nq) return;
    const float* xq = a.xq + q * kTcDim;
    float qn2 = 0.f;
    for (int t = lane; t < kTcDim; t += 32) qn2 = fmaf(xq[t], xq[t], qn2);
    for (int o = 16; o > 0; o >>= 1) qn2 += __shfl_xor_sync(0xffffffffu, qn2, o);
    const float cmax = a.cD[q * a.nprobe + a.nprobe - 1];
    if (!(cmax < 1.0e8f) || !(cmax >= 0.f) || !(qn2 < 1.0e30f)) {     // |q - c| may leave the fp16 range
        if (lane == 0) tau[q] = -kPosInf;
        return;
    }
    int64_t lst[2], beg[2] = {0, 0};
    int len[2] = {0, 0};
    float cdp[2] = {0.f, 0.f};
    for (int p = 0; p < 2; ++p) {
        lst[p] = p < a.nprobe ? cI[q * a.nprobe + p] : -1;
        if (lst[p] >= 0) {
            beg[p] = a.offsets[lst[p]];
            len[p] = static_cast<int>(a.lens[lst[p]]);
            const float cd = a.cD[q * a.nprobe + p];
            cdp[p] = cd + pair_err(cd, a.cb_bound);
            for (int t = lane; t < kTcDim; t += 32) s_x[warp][p][t] = xq[t] - a.centroids[lst[p] * kTcDim + t];
        }
    }
    if (len[0] >= 128) len[1] = 0;
    len[0] = min(len[0], kHeadMax);
    len[1] = min(len[1], kHeadMax - len[0]);
    const int total = len[0] + len[1];
    __syncwarp();
    for (int i = lane; i < total; i += 32) {
        const int p = i < len[0] ? 0 : 1;
        const int64_t slot = beg[p] + (p ? i - len[0] : i);
        const uint4 cw = unrotate_code(__ldg(reinterpret_cast<const uint4*>(a.codes + slot * 16)),
                                       static_cast<uint32_t>(slot & 15));
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
        const float* x = s_x[warp][p];
        float acc = 0.f, rn = 0.f;
#pragma unroll
        for (int m = 0; m < kTcM; ++m) {
            const uint32_t e = m * 256u + ((w[m >> 2] >> ((m & 3) * 8)) & 0xFFu);
            const uint4 hv = __ldg(reinterpret_cast<const uint4*>(a.cb16) + e);
            const float4 x0 = *reinterpret_cast<const float4*>(x + m * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(x + m * 8 + 4);
            const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&hv.x));
            const float2 r1 = __half22float2(*reinterpret_cast<const __half2*>(&hv.y));
            const float2 r2 = __half22float2(*reinterpret_cast<const __half2*>(&hv.z));
            const float2 r3 = __half22float2(*reinterpret_cast<const __half2*>(&hv.w));
            acc = fmaf(x0.x, r0.x, acc); acc = fmaf(x0.y, r0.y, acc);
            acc = fmaf(x0.z, r1.x, acc); acc = fmaf(x0.w, r1.y, acc);
            acc = fmaf(x1.x, r2.x, acc); acc = fmaf(x1.y, r2.y, acc);
            acc = fmaf(x1.z, r3.x, acc); acc = fmaf(x1.w, r3.y, acc);
            rn += __ldg(a.cbnorm + e);
        }
        s_v[warp][i] = order_bits(cdp[p] + fmaf(-2.f, acc, rn));
    }
    __syncwarp();
    float out = kPosInf;
    if (total >= kTcKeep) {
        // radix select of the value of rank k' - 1 among the ordered keys
        uint32_t prefix = 0, rank = kTcKeep - 1;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t hi_mask = bit == 31 ? 0u : ~((2u << bit) - 1u);
            uint32_t c0 = 0;
            for (int i = lane; i < total; i += 32) {
                const uint32_t v = s_v[warp][i];
                c0 += ((v & hi_mask) == prefix && !((v >> bit) & 1u)) ? 1u : 0u;
            }
            c0 = __reduce_add_sync(0xffffffffu, c0);
            if (rank >= c0) {
                rank -= c0;
                prefix |= 1u << bit;
            }
        }
        const float th = unorder_bits(prefix);
        const float bound = fabsf(cmax) + t2_bound + 2.f * sqrtf(qn2) * a.cb_bound + fabsf(th);
        out = th + 2.02f * err_rel * bound;
    }
    if (lane == 0) tau[q] = out;
}

__global__ void tc_order_keys_kernel(const int32_t* first, const int32_t* last, int nlist, int32_t* keys,
                                     int32_t* vals) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= nlist) return;
    keys[l] = 0x40000000 - (last[l] - first[l]);      // ascending sort: most queries first
    vals[l] = l;
}

__global__ void tc_cb16_kernel(const float* cb, int64_t n, uint16_t* out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half_as_ushort(__float2half_rn(cb[i]));
}

// ---------------------------------------------------------------------------------------
// selection of the k' best candidates of every query (one warp per query)
// ---------------------------------------------------------------------------------------
template <int PER_LANE>
__global__ void tc_select_kernel(const TcScanArgs a, float* fd, uint32_t* fp, float* fth) {
    const int64_t q = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (q >= a.nq) return;
    const unsigned int n_all = a.cand_n[q];
    const int n = static_cast<int>(n_all < static_cast<unsigned int>(a.cap) ? n_all : a.cap);
    unsigned long long key[PER_LANE];
#pragma unroll
    for (int s = 0; s < PER_LANE; ++s) {
        const int i = s * 32 + lane;
        key[s] = ~0ull;
        if (i < n) {
            const float dd = a.cand_d[q * a.cap + i];
            const uint32_t pp = a.cand_p[q * a.cap + i];
            key[s] = (static_cast<unsigned long long>(order_bits(dd)) << 32) | pp;
        }
    }
    unsigned long long mine = ~0ull;      // lane r ends up with the r-th smallest key
    for (int r = 0; r < kTcKeep; ++r) {
        unsigned long long m = key[0];
#pragma unroll
        for (int s = 1; s < PER_LANE; ++s) m = key[s] < m ? key[s] : m;
        unsigned long long w = m;
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, w, o);
            w = other < w ? other : w;
        }
        if (r == lane) mine = w;
        if (w == ~0ull) break;
        // remove one instance of the minimum (the lowest lane that holds it)
        const unsigned int holders = __ballot_sync(0xffffffffu, m == w);
        if (lane == __ffs(holders) - 1) {
            bool done = false;
#pragma unroll
            for (int s = 0; s < PER_LANE; ++s)
                if (!done && key[s] == w) {
                    key[s] = ~0ull;
                    done = true;
                }
        }
    }
    const bool have = mine != ~0ull;
    fp[q * kTcKeep + lane] = have ? static_cast<uint32_t>(mine & 0xFFFFFFFFull) : kNoPosTc;
    fd[q * kTcKeep + lane] = have ? unorder_bits(static_cast<uint32_t>(mine >> 32)) : kPosInf;
    const unsigned long long worst = __shfl_sync(0xffffffffu, mine, kTcKeep - 1);
    if (lane == 0) {
        const float t = a.tau[q];
        float th;
        if (n_all > static_cast<unsigned int>(a.cap) || t == -kPosInf) th = -kPosInf;       // candidates lost: exact path
        else if (worst != ~0ull) th = unorder_bits(static_cast<uint32_t>(worst >> 32));     // k' kept: the worst of them
        else th = t;                                    // fewer than k' emitted: everything else lies above tau
        fth[q] = th;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// the scan kernel: persistent, one CTA per SM.
//   warps 0-7  ("main"): decode a tile of 128 codes into shared memory, hand it to the MMA warp,
//              then run the epilogue of the PREVIOUS tile while the tensor core works -- one
//              continuous stream of tiles across lists.
//   warp 10    one thread issues the 16 UMMAs of every tile (two fp16 terms x K = 128).
//   warps 8, 9 ("scouts"): each prepares the next (list, query chunk) context of its own slot --
//              list from the global counter, column arrays, (q - c) rows as two fp16 terms in
//              UMMA layout -- while the main warps work through the other slot.
// ---------------------------------------------------------------------------------------
namespace {

constexpr int kAtomBytes = 128 * 128;            // A: 128 rows x 128 B (64 fp16 of K), SWIZZLE_128B
constexpr int kABytes = 2 * kAtomBytes;          // decoded tile: dims 0..63 | dims 64..127
constexpr int kBAtomBytes = kTcMaxN * 128;       // B: kTcMaxN rows x 128 B
constexpr int kBBytes = 4 * kBAtomBytes;         // query rows: high term (2 atoms) | low term (2 atoms)
constexpr int kCbBytes = kTcM * 256 * 16;        // fp16 codebooks, 16 B per codeword
constexpr int kCbnBytes = kTcM * 256 * 4;
constexpr int kColBytes = 3 * kTcMaxN * 4;       // per context: u[], cd[], q[]
constexpr int kOffA = 0;                         // two tiles
constexpr int kOffB = kOffA + 2 * kABytes;       // two contexts
constexpr int kOffCb = kOffB + 2 * kBBytes;
constexpr int kOffCbn = kOffCb + kCbBytes;
constexpr int kOffCol = kOffCbn + kCbnBytes;     // two contexts
constexpr int kOffRn = kOffCol + 2 * kColBytes;  // float [4][2][128] |r|^2 halves of the tiles in flight
constexpr int kTcSmemBytes = kOffRn + 4 * 2 * 128 * 4 + 1024;   // + room to align to 1024 B
constexpr uint32_t kTcTmemCols = 2 * kTcMaxN;    // two accumulators

constexpr uint32_t kTileStop = 0xFFFFFFFFu;

struct TcCtx {
    long long begin;   // first slot of the list
    int len;           // vectors in the list
    int cnt;           // queries (columns) of this chunk
    int done;          // 1: the scout of this slot has no more work
};

// byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled atom
__device__ __forceinline__ uint32_t sw_off(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return static_cast<uint32_t>(__half_as_ushort(a)) | (static_cast<uint32_t>(__half_as_ushort(b)) << 16);
}
__device__ __forceinline__ void main_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(kTcMainThreads) : "memory");
}

// One scout warp: fills context slot `slot` again and again until the list counter runs out.
__device__ __forceinline__ void scout_loop(const TcScanArgs& a, uint8_t* sm, int slot, int lane, TcCtx* ctx,
                                           uint64_t* ctx_full, uint64_t* ctx_free, volatile int* abort_flag) {
    float* s_u = reinterpret_cast<float*>(sm + kOffCol + slot * kColBytes);
    float* s_cd = s_u + kTcMaxN;
    int* s_q = reinterpret_cast<int*>(s_cd + kTcMaxN);
    uint8_t* bbase = sm + kOffB + slot * kBBytes;
    unsigned long long visited = 0;
    int f = 0, np = 0, c0 = 0, len = 0;
    long long list = -1, begin = 0;
    for (uint32_t it = 0;; ++it) {
        // next (list, chunk) and its column values: registers only, so all of this overlaps the wait
        // for the slot
        while (c0 >= np) {                          // next list with work
            unsigned int l = 0;
            if (lane == 0) l = atomicAdd(a.work, 1u);
            l = __shfl_sync(0xffffffffu, l, 0);
            if (l >= static_cast<unsigned int>(a.nlist)) {
                list = -1;
                break;
            }
            if (a.order) l = static_cast<unsigned int>(a.order[l]);
            list = l;
            f = a.first[l];
            np = a.last[l] - f;
            len = static_cast<int>(a.lens[l]);
            begin = a.offsets[l];
            c0 = 0;
            if (np <= 0 || len <= 0) {
                np = 0;
                continue;
            }
            visited += static_cast<unsigned long long>(np) * static_cast<unsigned long long>(len);
            const uint8_t* cp = a.codes + begin * 16;   // bring the list's codes into L2 ahead of the main warps
            for (int off = lane * 128; off < len * 16; off += 32 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(cp + off));
        }
        const bool have = list >= 0;
        const int cnt = have ? min(kTcMaxN, np - c0) : 0;
        const int n_mma = (cnt + 15) & ~15;
        int rq[kTcMaxN / 32];
        float rcd[kTcMaxN / 32], ru[kTcMaxN / 32];
#pragma unroll
        for (int r = 0; r < kTcMaxN / 32; ++r) {
            const int j = lane + 32 * r;
            rq[r] = 0;
            rcd[r] = 0.f;
            ru[r] = -kPosInf;
            if (j < cnt) {
                const int pair = a.sorted_pair[f + c0 + j];
                const int q = pair / a.nprobe;
                const float cd0 = a.cD[pair];
                const float cd = cd0 - pair_err(cd0, a.cb_bound);   // what leaves the epilogue is a lower bound
                rq[r] = q;
                rcd[r] = cd;
                ru[r] = a.tau[q] - cd;
            }
        }
        float4 e0 = make_float4(0.f, 0.f, 0.f, 0.f), e1 = e0;      // this lane's 8 dims of the centroid
        if (have) {
            const float4* cp = reinterpret_cast<const float4*>(a.centroids + list * kTcDim + (lane & 15) * 8);
            e0 = __ldg(cp);
            e1 = __ldg(cp + 1);
        }
        if (!ptx::mbar_wait_bounded(ctx_free, (it & 1u) ^ 1u, abort_flag)) break;
        if (!have) {
            if (lane == 0) {
                ctx->done = 1;
                ptx::mbar_arrive(ctx_full);
            }
            break;
        }
#pragma unroll
        for (int r = 0; r < kTcMaxN / 32; ++r) {
            s_q[lane + 32 * r] = rq[r];
            s_cd[lane + 32 * r] = rcd[r];
            s_u[lane + 32 * r] = ru[r];
        }
        __syncwarp();
        // (q - c) rows as fp16 high + low terms; a lane keeps one 16-byte chunk (8 dims) and walks the rows
        // The loads of eight rows are issued together, ahead of the conversions and stores: a load
        // that follows a shared-memory store in program order would wait for it.
        const int c = lane & 15;
        for (int j0 = lane >> 4; j0 < n_mma; j0 += 16) {
            float4 x0[8], x1[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int j = j0 + 2 * k;
                x0[k] = x1[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j < cnt) {
                    const float4* xp = reinterpret_cast<const float4*>(a.xq + static_cast<int64_t>(s_q[j]) * kTcDim + c * 8);
                    x0[k] = __ldg(xp);
                    x1[k] = __ldg(xp + 1);
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int j = j0 + 2 * k;
                if (j >= n_mma) break;
                uint4 hi = make_uint4(0, 0, 0, 0), lo = make_uint4(0, 0, 0, 0);
                if (j < cnt) {
                    const float v[8] = {x0[k].x - e0.x, x0[k].y - e0.y, x0[k].z - e0.z, x0[k].w - e0.w,
                                        x1[k].x - e1.x, x1[k].y - e1.y, x1[k].z - e1.z, x1[k].w - e1.w};
                    __half h[8], l[8];
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        h[t] = __float2half_rn(v[t]);
                        l[t] = __float2half_rn(v[t] - __half2float(h[t]));
                    }
                    hi = make_uint4(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]), pack_h2(h[4], h[5]), pack_h2(h[6], h[7]));
                    lo = make_uint4(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]), pack_h2(l[4], l[5]), pack_h2(l[6], l[7]));
                }
                const uint32_t off = sw_off(static_cast<uint32_t>(j), static_cast<uint32_t>(c & 7));
                *reinterpret_cast<uint4*>(bbase + (c >> 3) * kBAtomBytes + off) = hi;
                *reinterpret_cast<uint4*>(bbase + (2 + (c >> 3)) * kBAtomBytes + off) = lo;
            }
        }
        if (lane == 0) {
            ctx->begin = begin;
            ctx->len = len;
            ctx->cnt = cnt;
            ctx->done = 0;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ctx_full);
        c0 += kTcMaxN;
    }
    if (lane == 0 && visited) atomicAdd(a.scanned, visited);
}

__global__ void __launch_bounds__(kTcThreads, 1) ivfpq_tc_scan_kernel(const TcScanArgs a) {
    extern __shared__ uint8_t tc_raw[];
    uint8_t* sm = tc_raw + ((1024u - (ptx::smem_u32(tc_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t mbar[2];        // MMAs of the tile in accumulator / A buffer b are complete
    __shared__ __align__(8) uint64_t ctx_full[2];    // scout -> main: context slot filled
    __shared__ __align__(8) uint64_t ctx_free[2];    // main -> scout: context slot may be refilled
    __shared__ __align__(8) uint64_t a_full[2];      // main -> MMA warp: tile decoded into A buffer b
    __shared__ uint32_t tile_info[2];                // its UMMA N | context slot << 16; kTileStop: no more tiles
    __shared__ TcCtx ctx[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ unsigned int s_stage_n;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < kCbBytes / 16; i += kTcThreads)
        reinterpret_cast<uint4*>(sm + kOffCb)[i] = reinterpret_cast<const uint4*>(a.cb16)[i];
    for (int i = tid; i < kCbnBytes / 16; i += kTcThreads)
        reinterpret_cast<uint4*>(sm + kOffCbn)[i] = reinterpret_cast<const uint4*>(a.cbnorm)[i];
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&mbar[i], 1);
            ptx::mbar_init(&ctx_full[i], 1);
            ptx::mbar_init(&ctx_free[i], 1);
            ptx::mbar_init(&a_full[i], kTcMainThreads);
        }
        abort_flag = 0;
        s_stage_n = 0;
        ptx::mbar_fence_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(&tmem_slot, kTcTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == kTcMainThreads / 32 + 2) {
        // ---- MMA warp: one thread issues the 16 UMMAs of every decoded tile ----
        if (lane == 0) {
            const uint64_t desc_hi = ptx::umma_desc_k_sw128(0);
            const uint32_t a_lo = (ptx::smem_u32(sm + kOffA) & 0x3FFFFu) >> 4;
            const uint32_t b_lo = (ptx::smem_u32(sm + kOffB) & 0x3FFFFu) >> 4;
            for (uint32_t gm = 0;; ++gm) {
                const uint32_t buf = gm & 1u;
                if (!ptx::mbar_wait_bounded(&a_full[buf], (gm >> 1) & 1u, &abort_flag)) break;
                const uint32_t info = tile_info[buf];
                if (info == kTileStop) break;
                ptx::tc_fence_after();
                const uint32_t idesc = ptx::umma_idesc(1, 0, kTcTile, info & 0xFFFFu);
                const uint32_t tacc = tmem_base + buf * kTcMaxN;
                const uint32_t at_lo = a_lo + buf * (kABytes >> 4);
                const uint32_t bs_lo = b_lo + (info >> 16) * (kBBytes >> 4);
#pragma unroll
                for (uint32_t prod = 0; prod < 2; ++prod)
#pragma unroll
                    for (uint32_t at = 0; at < 2; ++at)
#pragma unroll
                        for (uint32_t ks = 0; ks < 4; ++ks) {
                            const uint64_t da = desc_hi | static_cast<uint64_t>(at_lo + at * (kAtomBytes >> 4) + ks * 2);
                            const uint64_t db = desc_hi | static_cast<uint64_t>(bs_lo + (prod * 2 + at) * (kBAtomBytes >> 4) + ks * 2);
                            ptx::umma_f16(tacc, da, db, idesc, (prod | at | ks) ? 1u : 0u);
                        }
                ptx::umma_commit(&mbar[buf]);
            }
        }
    } else if (warp >= kTcMainThreads / 32) {
        const int slot = warp - kTcMainThreads / 32;
        scout_loop(a, sm, slot, lane, &ctx[slot], &ctx_full[slot], &ctx_free[slot], &abort_flag);
    } else {
        const uint32_t row = tid & 127, half = tid >> 7;
        const uint32_t quarter = warp & 3, cb0 = warp >> 2;
        float* s_rn = reinterpret_cast<float*>(sm + kOffRn);
        const float* s_cbn = reinterpret_cast<const float*>(sm + kOffCbn);

        uint32_t g = 0;                        // tiles issued so far: buffers g & 1, phase (g >> 1) & 1
        uint32_t uses0 = 0, uses1 = 0;         // contexts consumed per slot
        int done_mask = 0, slot = 0;
        bool aborted = false;
        // the tile whose epilogue is still to run
        bool pend = false, p_last = false;
        int p_slot = 0, p_tile = 0, p_len = 0, p_nld = 0;
        long long p_begin = 0;

        const bool prof_on = a.prof != nullptr && tid == 0;
        long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // ctx wait, decode, barrier, issue, mma wait, epilogue, release, tiles
        // The epilogue of a tile in two steps.  epi_load brings the warp's 32 accumulator columns
        // into registers and must run BEFORE the next tile is handed to the MMA warp: a TMEM load
        // issued behind 16 queued UMMAs waits for them.  epi_compute works on the registers while
        // the tensor core runs.  (kTcMaxN = 64: a warp owns at most one block of 32 columns.)
        uint32_t acc[32];
        bool acc_ok = false;
        auto epi_load = [&](uint32_t ge) {
            acc_ok = false;
            const uint32_t buf = ge & 1u;
            const long long w0 = prof_on ? clock64() : 0;
            if (!ptx::mbar_wait_bounded(&mbar[buf], (ge >> 1) & 1u, &abort_flag)) return;
            if (prof_on) pc[4] += clock64() - w0;
            ptx::tc_fence_after();
            if (static_cast<int>(cb0) * 32 < p_nld) {
                ptx::tmem_ld_32x32(tmem_base + buf * kTcMaxN + cb0 * 32 + ((quarter * 32u) << 16), acc);
                ptx::tmem_ld_wait(acc);
                acc_ok = true;
            }
            ptx::tc_fence_before();
        };
        auto epi_compute = [&](uint32_t ge) {
            if (!acc_ok) return;
            const float* s_u = reinterpret_cast<const float*>(sm + kOffCol + p_slot * kColBytes);
            const float* s_cd = s_u + kTcMaxN;
            const int* s_q = reinterpret_cast<const int*>(s_cd + kTcMaxN);
            const int rr = p_tile * kTcTile + static_cast<int>(row);
            const bool valid = rr < p_len;
            const float rn = s_rn[(ge & 3u) * 256 + row] + s_rn[(ge & 3u) * 256 + 128 + row];
            const uint32_t pos = static_cast<uint32_t>(p_begin + rr);
            const int b = static_cast<int>(cb0);
            const float4* up = reinterpret_cast<const float4*>(s_u + b * 32);
            uint32_t hits = 0;                 // bit j: column j of the block passes
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                const float4 u = up[j4];
                hits |= (fmaf(-2.f, __uint_as_float(acc[4 * j4 + 0]), rn) <= u.x ? 1u : 0u) << (4 * j4 + 0);
                hits |= (fmaf(-2.f, __uint_as_float(acc[4 * j4 + 1]), rn) <= u.y ? 1u : 0u) << (4 * j4 + 1);
                hits |= (fmaf(-2.f, __uint_as_float(acc[4 * j4 + 2]), rn) <= u.z ? 1u : 0u) << (4 * j4 + 2);
                hits |= (fmaf(-2.f, __uint_as_float(acc[4 * j4 + 3]), rn) <= u.w ? 1u : 0u) << (4 * j4 + 3);
            }
            if (!valid) hits = 0;
            // rare: about one pair in a thousand passes.  The accumulator of a hit is fetched from the
            // register array through a select chain only here.
            while (hits) {
                const int j = __ffs(hits) - 1;
                hits &= hits - 1;
                float av = 0.f;
#pragma unroll
                for (int t = 0; t < 32; ++t) av = t == j ? __uint_as_float(acc[t]) : av;
                const int col = b * 32 + j;
                const float v = fmaf(-2.f, av, rn);
                // staged per CTA (shared-memory counter, one 16-byte store): the per-query slots are
                // handed out later by tc_scatter_kernel, where the round trip of a global atomic does
                // not stall an epilogue warp
                const unsigned int sl = atomicAdd(&s_stage_n, 1u);
                if (sl < static_cast<unsigned int>(a.stage_cap)) {
                    a.stage[static_cast<size_t>(blockIdx.x) * a.stage_cap + sl] =
                        make_uint4(static_cast<uint32_t>(s_q[col]), pos, __float_as_uint(s_cd[col] + v), 0u);
                } else {                            // staging area full: append directly
                    const int64_t q = s_q[col];
                    const unsigned int qs = atomicAdd(a.cand_n + q, 1u);
                    if (qs < static_cast<unsigned int>(a.cap)) {
                        a.cand_d[q * a.cap + qs] = s_cd[col] + v;
                        a.cand_p[q * a.cap + qs] = pos;
                    }
                }
            }
        };
        auto epilogue = [&]() {            // both steps, for the pending tile g - 1
            epi_load(g - 1);
            epi_compute(g - 1);
        };

        while (!aborted) {
            if (done_mask == 3) break;
            if (done_mask & (1 << slot)) slot ^= 1;
            if (pend && p_slot == slot) {
                // the slot to be waited for is still held by the pending tile (only the other scout has
                // run out of work): finish that tile first, or its scout could never refill the slot
                epilogue();
                main_barrier();
                if (tid == 0) ptx::mbar_arrive(&ctx_free[p_slot]);
                pend = false;
                if (abort_flag) { aborted = true; break; }
            }
            const uint32_t use = slot ? uses1 : uses0;
            const long long cw0 = prof_on ? clock64() : 0;
            if (!ptx::mbar_wait_bounded(&ctx_full[slot], use & 1u, &abort_flag)) { aborted = true; break; }
            if (prof_on) pc[0] += clock64() - cw0;
            if (slot) ++uses1; else ++uses0;
            if (ctx[slot].done) {
                done_mask |= 1 << slot;
                slot ^= 1;
                continue;
            }
            const long long begin = ctx[slot].begin;
            const int len = ctx[slot].len, cnt = ctx[slot].cnt;
            const int n_mma = (cnt + 15) & ~15, n_ld = (cnt + 31) & ~31;
            const int padded = (len + 31) & ~31;
            const int ntiles = (len + kTcTile - 1) / kTcTile;

            auto load_code = [&](int tile) {
                const int r0 = tile * kTcTile + static_cast<int>(row);
                uint4 cw = make_uint4(0, 0, 0, 0);
                if (tile < ntiles && r0 < padded) cw = __ldg(reinterpret_cast<const uint4*>(a.codes + (begin + r0) * 16));
                return cw;
            };
            uint4 cw = load_code(0);
            for (int t = 0; t < ntiles; ++t) {
                const uint32_t buf = g & 1u;
                const long long d0 = prof_on ? clock64() : 0;
                {   // decode tile t into A[buf]: one 16-byte codeword per sub-quantizer, 8 sub-quantizers per thread
                    const uint4 cc = unrotate_code(cw, static_cast<uint32_t>((begin + t * kTcTile + row) & 15));
                    const uint32_t lo_w = half ? cc.z : cc.x, hi_w = half ? cc.w : cc.y;
                    uint8_t* arow = sm + kOffA + buf * kABytes + half * kAtomBytes + (row >> 3) * 1024u + (row & 7u) * 128u;
                    const uint8_t* cbm = sm + kOffCb + half * 8u * 256u * 16u;
                    const float* cbn = s_cbn + half * 8u * 256u;
                    float rn = 0.f;
                    uint4 v[8];                      // all lookups first, then the stores
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        const uint32_t byte = ((i < 4 ? lo_w : hi_w) >> ((i & 3u) * 8u)) & 0xFFu;
                        const uint32_t e = i * 256u + byte;
                        v[i] = *reinterpret_cast<const uint4*>(cbm + e * 16u);
                        rn += cbn[e];
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(arow + ((i ^ (row & 7u)) << 4)) = v[i];
                    s_rn[(g & 3u) * 256 + half * 128 + row] = rn;
                }
                const long long d1 = prof_on ? clock64() : 0;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                ptx::tc_fence_before();
                main_barrier();
                const long long d2 = prof_on ? clock64() : 0;
                if (abort_flag) { aborted = true; break; }
                if (pend) epi_load(g - 1);           // before the UMMAs of this tile enter the pipe
                if (tid == 0) tile_info[buf] = static_cast<uint32_t>(n_mma) | (static_cast<uint32_t>(slot) << 16);
                ptx::mbar_arrive(&a_full[buf]);      // every main thread: its rows are written and its load is done
                ++g;
                const long long d3 = prof_on ? clock64() : 0;
                cw = load_code(t + 1);               // in flight behind the epilogue
                if (pend) {
                    epi_compute(g - 2);
                    const long long d4 = prof_on ? clock64() : 0;
                    if (p_last) {                    // the context of the pending tile is finished: hand its slot back
                        main_barrier();
                        if (tid == 0) ptx::mbar_arrive(&ctx_free[p_slot]);
                    }
                    if (prof_on) {
                        pc[5] += d4 - d3;
                        pc[6] += clock64() - d4;
                    }
                }
                if (prof_on) {
                    pc[1] += d1 - d0;
                    pc[2] += d2 - d1;
                    pc[3] += d3 - d2;
                    pc[7] += 1;
                }
                pend = true;
                p_last = t + 1 == ntiles;
                p_slot = slot;
                p_tile = t;
                p_len = len;
                p_nld = n_ld;
                p_begin = begin;
            }
            slot ^= 1;
        }
        if (pend && !aborted) {
            epilogue();
            main_barrier();
            if (tid == 0 && p_last) ptx::mbar_arrive(&ctx_free[p_slot]);
        }
        if (tid == 0) tile_info[g & 1u] = kTileStop;     // release the MMA warp
        ptx::mbar_arrive(&a_full[g & 1u]);
        if (prof_on)
            for (int i = 0; i < 8; ++i) atomicAdd(a.prof + i, static_cast<unsigned long long>(pc[i]));
    }

    __syncwarp();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTcTmemCols);
    }
    if (tid == 0) {
        a.stage_n[blockIdx.x] = s_stage_n;
        if (abort_flag) atomicOr(a.err, 1u);
    }
}

// Moves the staged candidates of CTA blockIdx.x into the per-query arrays.
__global__ void tc_scatter_kernel(const TcScanArgs a) {
    // entries beyond the staging capacity were appended by the scan kernel itself
    const unsigned int n_all = min(a.stage_n[blockIdx.x], static_cast<unsigned int>(a.stage_cap));
    const uint4* st = a.stage + static_cast<size_t>(blockIdx.x) * a.stage_cap;
    for (unsigned int i = threadIdx.x; i < n_all; i += blockDim.x) {
        const uint4 e = st[i];
        const int64_t q = e.x;
        const unsigned int sl = atomicAdd(a.cand_n + q, 1u);
        if (sl < static_cast<unsigned int>(a.cap)) {
            a.cand_d[q * a.cap + sl] = __uint_as_float(e.z);
            a.cand_p[q * a.cap + sl] = e.y;
        }
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
namespace {
inline unsigned int blocks(int64_t n, int per) { return static_cast<unsigned int>((n + per - 1) / per); }
}  // namespace

cudaError_t launch_tc_keys(const int64_t* cI, int64_t npairs, int nlist, int32_t* keys, int32_t* vals,
                           cudaStream_t st) {
    tc_keys_kernel<<<blocks(npairs, 256), 256, 0, st>>>(cI, npairs, nlist, keys, vals);
    return cudaGetLastError();
}

cudaError_t launch_tc_bounds(const int32_t* sorted_keys, int64_t npairs, int nlist, int32_t* first, int32_t* last,
                             cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(first, 0, static_cast<size_t>(nlist) * 4, st);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(last, 0, static_cast<size_t>(nlist) * 4, st);
    if (e != cudaSuccess) return e;
    tc_bounds_kernel<<<blocks(npairs, 256), 256, 0, st>>>(sorted_keys, npairs, nlist, first, last);
    return cudaGetLastError();
}

cudaError_t launch_tc_head_tau(const TcScanArgs& a, const int64_t* cI, float err_rel, float t2_bound, float* tau,
                               cudaStream_t st) {
    tc_head_tau_kernel<<<blocks(a.nq, kHeadWarps), kHeadWarps * 32, 0, st>>>(a, cI, err_rel, t2_bound, tau);
    return cudaGetLastError();
}

cudaError_t launch_tc_order_keys(const int32_t* first, const int32_t* last, int nlist, int32_t* keys, int32_t* vals,
                                 cudaStream_t st) {
    tc_order_keys_kernel<<<blocks(nlist, 256), 256, 0, st>>>(first, last, nlist, keys, vals);
    return cudaGetLastError();
}

cudaError_t launch_tc_scan(const TcScanArgs& a, int num_sms, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(a.work, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(a.cand_n, 0, static_cast<size_t>(a.nq) * sizeof(unsigned int), st);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(ivfpq_tc_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
    if (e != cudaSuccess) return e;
    ivfpq_tc_scan_kernel<<<num_sms, kTcThreads, kTcSmemBytes, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    tc_scatter_kernel<<<num_sms, 512, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_tc_select(const TcScanArgs& a, float* fd, uint32_t* fp, float* fth, cudaStream_t st) {
    if (a.cap == 256) tc_select_kernel<8><<<blocks(a.nq, 8), 256, 0, st>>>(a, fd, fp, fth);
    else if (a.cap == 128) tc_select_kernel<4><<<blocks(a.nq, 8), 256, 0, st>>>(a, fd, fp, fth);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_tc_cb16(const float* cb, int64_t n, uint16_t* out, cudaStream_t st) {
    tc_cb16_kernel<<<blocks(n, 256), 256, 0, st>>>(cb, n, out);
    return cudaGetLastError();
}

}  // namespace b200
