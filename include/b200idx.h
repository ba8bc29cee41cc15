/*
 * b200idx -- C ABI of the B200-native search hot path (Flat / Int8Flat / IVFPQ search and
 * multi-index batch search).  Plain pointers and sizes only; no C++ types, no exceptions.
 * Every entry point returns an APP_ERROR-compatible int (0 = OK) and records a message that
 * b200idx_last_error() returns.
 *
 * Each declaration names the interface of the reference (Ascend/IndexSDK) it stands in for.
 * FR = feature_retrieval/src/ascendfaiss.
 */
#ifndef B200IDX_H
#define B200IDX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200idx_index b200idx_t;

/* Status codes: FR/common/ErrorCode.h:50-66 (APP_ERR_OK, APP_ERR_INVALID_PARAM,
 * APP_ERR_NOT_IMPLEMENT, APP_ERR_INNER_ERROR, APP_ERR_TIMEOUT). */
enum {
    B200IDX_OK = 0,
    B200IDX_ERR_INVALID_PARAM = 2001,
    B200IDX_ERR_NOT_IMPLEMENTED = 2008,
    B200IDX_ERR_INNER = 2010,
    B200IDX_ERR_TIMEOUT = 2011
};

/* Metric values mirror the device layer of the reference: FR/ascenddaemon/impl/Index.h:60-64. */
enum {
    B200IDX_METRIC_INNER_PRODUCT = 0,
    B200IDX_METRIC_L2 = 1,
    /* Int8Flat only: the fp16 cosine the reference's Int8Flat index returns for
     * METRIC_INNER_PRODUCT (FR/ascend/impl/AscendIndexInt8FlatImpl.cpp:790-793 instantiates the
     * "Cos" index; arithmetic of FR/ops/tbe/impl/int8_l2_norm.py:140-183 and
     * FR/ops/tbe/impl/distance_int8_cos_maxs.py:256-284):
     *   fp16( fp16(q.x * 0.01) * fp16( rnorm(x) * rnorm(q) ) ),  rnorm(v) = fp16(1 / sqrt(fp16(|v|^2 * 0.01)));
     * larger is better, ties by lower position, a NaN score ranks last and is reported as -inf.
     * B200IDX_METRIC_INNER_PRODUCT on an Int8Flat index stays the exact int32 dot product. */
    B200IDX_METRIC_INT8_COSINE = 2
};

/* Storage / arithmetic type of a Flat index.
 *   F32: fp32 rows; a bf16 tensor-core pass filters candidates, results are re-computed in fp32.
 *   F16: fp16 rows, fp32 accumulation (the reference's own Flat arithmetic,
 *        FR/ascend/impl/AscendIndexImpl.cpp:339-346). */
enum { B200IDX_F32 = 0, B200IDX_F16 = 1 };

/* ---- construction: AscendIndexFlat(int dims, MetricType, AscendIndexFlatConfig)
 *      FR/ascend/AscendIndexFlat.h:56; AscendIndexInt8Flat(...) FR/ascend/AscendIndexInt8Flat.h:63-64;
 *      AscendIndexIVFPQ(dims, metric, nlist, msubs, nbits, config) FR/ascend/AscendIndexIVFPQ.h:74-75.
 *      One handle lives on one CUDA device (an entry of the reference's deviceList). ---- */
int b200idx_create_flat(int d, int metric, int dtype, int device, b200idx_t** out);
int b200idx_create_int8flat(int d, int metric, int device, b200idx_t** out);
int b200idx_create_ivfpq(int d, int metric, int nlist, int M, int nbits, int by_residual, int device,
                         b200idx_t** out);
/* ~AscendIndex(): FR/ascend/AscendIndex.h:66 */
int b200idx_destroy(b200idx_t* h);

/* ---- add / add_with_ids: FR/ascend/AscendIndex.h:70-74 (float), :103-105 (fp16 bits),
 *      FR/ascend/AscendIndexInt8.h:70-84 (int8).  x and ids are host pointers; ids may be NULL
 *      (labels become ntotal + i, FR/ascend/impl/AscendIndexImpl.h:59-83). ---- */
int b200idx_add(b200idx_t* h, int64_t n, const void* x, const int64_t* ids);
int b200idx_add_f16(b200idx_t* h, int64_t n, const uint16_t* x, const int64_t* ids);
/* Same with x resident on the index's device (no reference counterpart: the reference accepts
 * host pointers only; used to build large synthetic bases without a host round trip). */
int b200idx_add_device(b200idx_t* h, int64_t n, const void* x_dev, const int64_t* ids_host);

/* ---- search: FR/ascend/AscendIndex.h:80-82 (float), :107 (fp16), FR/ascend/AscendIndexInt8.h:93-96.
 *      Writes exactly n*k distances and labels; missing results are FLT_MAX / -1
 *      (FR/ascend/impl/AscendIndexImpl.cpp:628-633). ---- */
int b200idx_search(b200idx_t* h, int64_t n, const void* x, int k, float* distances, int64_t* labels);
int b200idx_search_f16(b200idx_t* h, int64_t n, const uint16_t* x, int k, float* distances, int64_t* labels);
/* Search restricted by a filter: `mask` holds n rows of ceil(ntotal / 8) bytes; bit (i % 8) of byte
 * i / 8 of a row is 1 when base position i (add order) may appear in that query's result (replaces
 * AscendIndexFlat::search_with_masks, feature_retrieval/src/ascendfaiss/ascend/AscendIndexFlat.h:78-82;
 * device predicate feature_retrieval/src/ascendfaiss/ops/ascendc/op_kernel/distance_flat_l2.cpp:487-533).
 * Flat and Int8Flat indexes; queries in the index's input dtype (float for F32 / F16 indexes). */
int b200idx_search_with_masks(b200idx_t* h, int64_t n, const void* x, int k, const uint8_t* mask, float* distances,
                              int64_t* labels);

/* Device-resident variant: x, distances, labels are device pointers on the index's device; the
 * call returns after the index's stream has been synchronised. */
int b200idx_search_device(b200idx_t* h, int64_t n, const void* x_dev, int k, float* distances_dev,
                          int64_t* labels_dev);

/* Device-resident exact search that allocates nothing (no counterpart in the reference, whose
 * operators always draw temporaries from a per-index pool).  For callers that may not allocate
 * device memory while searching -- a process whose HBM is owned by its own pool, or a loop that
 * cannot take the device-wide synchronisation of cudaMalloc / cudaFree.  Same kernels and same
 * results as b200idx_search_device on a Flat or Int8Flat index, with every scratch buffer taken
 * from one static device array of 10 MiB + 96 KiB: n * round_up(ntotal, 256) <= 2^20, k <= 1024,
 * n * k <= 131072, n * d <= 524288; anything larger returns B200IDX_ERR_INVALID_PARAM.  Calls
 * share that array: do not overlap two of them on one GPU.  The first call on a device resolves
 * the array's address and should be made before any stream capture. */
int b200idx_search_device_noalloc(b200idx_t* h, int64_t n, const void* x_dev, int k, float* distances_dev,
                                  int64_t* labels_dev);

/* ---- multi-index batch search: faiss::ascend::Search(indexes, n, x, k, D, I, merged),
 *      FR/ascend/AscendMultiIndexSearch.h:34-44, .cpp:230-324.  merged = 0: output layout
 *      [index][n][k]; merged = 1: [n][k] by (distance, label)
 *      (FR/ascend/utils/MergeResUtils.cpp:44-107).  Also serves base sets sharded over several
 *      devices (FR/ascend/impl/AscendIndexImpl.cpp:375-403,587-642). ---- */
int b200idx_search_multi(b200idx_t* const* hs, int nh, int64_t n, const void* x, int k, float* distances,
                         int64_t* labels, int merged);

/* Counters of the segmented path of b200idx_search_multi on one device: small Flat / Int8Flat
 * indexes of a device are searched in one pass over their concatenated bases, the counterpart of
 * the reference's single top-k operator over the blocks of all indexes
 * (FR/ops/cpukernel/impl/topk_multisearch_cpu_kernel.cpp:316-430).  group_launches: kernels
 * launched by that path so far (per call it does not depend on the number of indexes);
 * group_rebuilds: times the concatenated copy was (re)built -- it is kept until a member changes. */
int b200idx_search_multi_stats(int device, uint64_t* group_launches, uint64_t* group_rebuilds);

/* Merge of nsrc sorted per-shard results resident on one device: Din/Iin [nsrc][n][k] ->
 * D/I [n][k]; descending = 1 for inner-product scores.  Stands in for the host merge
 * FR/ascend/impl/AscendIndexImpl.cpp:587-642 after a gather of per-rank results.
 * stream: a cudaStream_t (NULL = default stream); asynchronous. */
int b200idx_merge_topk_device(int nsrc, int64_t n, int k, int descending, const float* Din_dev,
                              const int64_t* Iin_dev, float* D_dev, int64_t* I_dev, void* stream);

/* The same for sources that are src_stride_bytes apart (a multiple of 8): source s has its distances
 * at Din_dev + s * src_stride_bytes and its labels at Iin_dev + s * src_stride_bytes (byte offsets).
 * This is the layout one all-gather of packed per-rank blocks [n*k distances | n*k labels] leaves in
 * local memory, so the results of all ranks are exchanged with ONE collective and merged in place. */
int b200idx_merge_topk_device_strided(int nsrc, int64_t n, int k, int descending, const float* Din_dev,
                                      const int64_t* Iin_dev, int64_t src_stride_bytes, float* D_dev,
                                      int64_t* I_dev, void* stream);

/* ---- reset / remove_ids / bookkeeping: FR/ascend/AscendIndex.h:77,91;
 *      getBaseSize / getBase / getIdxMap FR/ascend/AscendIndexFlat.h:69-75,
 *      FR/ascend/AscendIndexInt8Flat.h:78-84. ---- */
int b200idx_reset(b200idx_t* h);
int b200idx_remove_ids(b200idx_t* h, int64_t n, const int64_t* ids, int64_t* n_removed);
int64_t b200idx_ntotal(const b200idx_t* h);
int b200idx_dim(const b200idx_t* h);
int b200idx_device(const b200idx_t* h);
/* rows [offset, offset+n): float (F32), fp16 bits (F16) or int8 */
int b200idx_get_base(const b200idx_t* h, int64_t offset, int64_t n, void* out);
int b200idx_get_ids(const b200idx_t* h, int64_t offset, int64_t n, int64_t* out);

/* ---- IVFPQ: trained state comes in the way copyFrom(const faiss::IndexIVFPQ*) brings it
 *      (FR/ascend/impl/AscendIndexIVFPQImpl.cpp:392-425): centroids [nlist][d], codebooks
 *      [M][256][d/M] (layout FR/ascend/impl/AscendIndexIVFPQImpl.h:158-159). ---- */
int b200idx_ivfpq_set_centroids(b200idx_t* h, const float* centroids);
int b200idx_ivfpq_set_codebooks(b200idx_t* h, const float* codebooks);
int b200idx_ivfpq_get_centroids(const b200idx_t* h, float* out);
int b200idx_ivfpq_get_codebooks(const b200idx_t* h, float* out);
/* pre-encoded vectors, e.g. the inverted lists of a CPU index (copyFrom) */
int b200idx_ivfpq_add_codes(b200idx_t* h, int64_t n, const int32_t* list_no, const uint8_t* codes,
                            const int64_t* ids);
/* setNumProbes / getNumProbes: FR/ascend/AscendIndexIVF.h:93-96 */
int b200idx_ivfpq_set_nprobe(b200idx_t* h, int nprobe);

/* Training on the device.  b200idx_kmeans: Lloyd k-means of n host vectors into k centroids (start:
 * centroid c = x[(floor(c n / k) + seed) mod n]; nearest centroid under the canonical fp32 L2
 * distance, ties to the lower centroid; mean of the members summed in fp64 in increasing vector
 * index; a centroid without members keeps its value).  b200idx_ivfpq_train: coarse centroids with
 * k = nlist, then one 256-entry codebook per sub-space (seed + 1 + m), on the residuals to the
 * assigned centroid when the index encodes residuals; the index must be empty.  Replaces the
 * reference's NPU training (feature_retrieval/src/ascendfaiss/ascenddaemon/impl/IndexIVFPQ.cpp:
 * 810-1135,1340-1430; ascend/impl/AscendIndexIVFPQImpl.cpp:962-1252). */
int b200idx_kmeans(int device, int d, int64_t n, const float* x, int k, int niter, uint64_t seed, float* centroids);
int b200idx_ivfpq_train(b200idx_t* h, int64_t n, const float* x, int niter, uint64_t seed);

/* The two halves of an IVFPQ search, device-resident (the reference runs them back to back inside
 * IndexIVFPQ::searchImpl: probe selection feature_retrieval/src/ascendfaiss/ascenddaemon/impl/
 * IndexIVFPQ.cpp:2104-2164, code scan + top-k :2165-2411).  Split so that the ranks of a sharded
 * index -- every rank holds the full coarse quantizer -- can each select the probes of a slice of
 * the queries, exchange them, and scan their shard for all queries.
 *   coarse      : probe_distances_dev / probe_lists_dev [n][nprobe] <- the nprobe nearest centroids
 *                 (canonical fp32 distances, ascending; list -1 = none)
 *   preassigned : searches the given probes; same results as b200idx_search_device when they come
 *                 from coarse on the same queries */
int b200idx_ivfpq_coarse_device(b200idx_t* h, int64_t n, const float* x_dev, float* probe_distances_dev,
                                int64_t* probe_lists_dev);
int b200idx_ivfpq_search_preassigned_device(b200idx_t* h, int64_t n, const float* x_dev, int k,
                                            const float* probe_distances_dev, const int64_t* probe_lists_dev,
                                            float* distances_dev, int64_t* labels_dev);
int b200idx_ivfpq_get_nprobe(const b200idx_t* h);
/* getListLength / getListCodesAndIds: FR/ascend/AscendIndexIVF.h:105-108 */
int64_t b200idx_ivfpq_list_length(const b200idx_t* h, int list);
int b200idx_ivfpq_get_list(const b200idx_t* h, int list, uint8_t* codes, int64_t* ids);

/* Persistence in this library's own file format: everything needed to search again -- vectors in the
 * index's storage dtype and labels (Flat, Int8Flat), or the trained state, list contents and nprobe
 * (IVFPQ).  Replaces the reference's route through a CPU Faiss index, index_ascend_to_cpu +
 * faiss::write_index / read_index + index_cpu_to_ascend (feature_retrieval/src/ascendfaiss/ascend/
 * AscendCloner.cpp:64-99,159-196,232-281).  load creates the index on `device`. */
int b200idx_save(const b200idx_t* h, const char* path);
int b200idx_load(const char* path, int device, b200idx_t** out);

/* ---- counters (the reference has none; APP_LOG timings only) ---- */
enum {
    B200IDX_STAGE_SAMPLE = 0,    /* query prep + sample GEMM pass + threshold selection */
    B200IDX_STAGE_FULL_GEMM = 1, /* full distance-GEMM pass with the append epilogue */
    B200IDX_STAGE_REFINE = 2,    /* fp32 re-computation of candidates */
    B200IDX_STAGE_SELECT = 3,    /* exact top-k of candidates + result emission */
    B200IDX_STAGE_COARSE = 4,    /* IVFPQ: whole coarse-quantizer search (host-side span) */
    B200IDX_STAGE_LUT = 5,       /* IVFPQ: lookup tables */
    B200IDX_STAGE_SCAN = 6,      /* IVFPQ: code scan */
    B200IDX_STAGE_MERGE = 7,     /* IVFPQ: merge of probe splits */
    B200IDX_NUM_STAGES = 8
};
typedef struct {
    double stage_ms[B200IDX_NUM_STAGES];        /* CUDA-event time per stage (timing enabled only) */
    uint64_t stage_launches[B200IDX_NUM_STAGES];
    uint64_t searches;
    uint64_t queries;
    uint64_t fallback_queries; /* queries re-run without a threshold after a candidate overflow (IVFPQ: exact re-scan) */
    uint64_t gemm_launches;
    uint64_t kernel_launches;  /* kernels of this library launched by searches */
    uint64_t scan_codes;       /* IVFPQ: PQ codes visited so far */
    uint64_t second_pass_queries; /* IVFPQ: queries whose first filter pass could not be verified (ties at its
                                     boundary) and that took the second, fixed-threshold filter pass */
} b200idx_stats_t;
int b200idx_stats(b200idx_t* h, b200idx_stats_t* out, int reset);
/* Per-stage CUDA-event timing on the index's stream (off by default; the reference only has
 * verbose wall-clock prints, FR/ascend/impl/AscendIndexIVFPQImpl.cpp:114-118). */
int b200idx_set_timing(b200idx_t* h, int enabled);
/* The cudaStream_t all of this index's kernels are launched on. */
void* b200idx_stream(const b200idx_t* h);

/* Message of the last failing call on this handle (h = NULL: last failing create). */
const char* b200idx_last_error(const b200idx_t* h);
/* The status code this library returns for an internal failure with the given message: a device-side
 * wait that ran out of its bound (the kernels give every mbarrier / flag wait a limit and report
 * through an error word) maps to B200IDX_ERR_TIMEOUT, anything else to B200IDX_ERR_INNER -- the
 * reference's APP_ERR_TIMEOUT for its bounded flag wait, FR/ops/cpukernel/impl/utils/kernel_utils.h:105-155,
 * FR/common/ErrorCode.h:62.  Host-only; lets the translation be checked without a device fault. */
int b200idx_status_of_message(const char* message);
const char* b200idx_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200IDX_H */
