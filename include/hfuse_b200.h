/*
 * hfuse_b200 — C ABI of the horizontally fused kernel pairs for NVIDIA B200 (sm_100a).
 *
 * The reference (aoli-al/HFuse) has a source-level boundary: it prints fused
 * `__global__` functions into `<K1>_<K2>_.inc` (tools/llvm-smart-fuser/main.cpp:247-257)
 * whose parameter list is K1's parameters followed by K2's
 * (lib/KernelFuser/KernelPrinter.cpp:107-114), and external host code launches them as
 * `<<<grid, T1+T2, shmem, stream>>>(args of K1..., args of K2...)`
 * (scripts/configs/hist_norm.json:5).  Each entry point below replaces one such launch
 * site: same argument order (K1's then K2's, then the stream), buffers owned by the
 * caller, results written in place, nothing allocated, nothing synchronised.
 *
 * Conventions
 *   - every pointer is a device pointer on the current CUDA device unless its comment
 *     says "host"; float buffers are contiguous NCHW fp32, 16-byte aligned;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream);
 *   - return value: HFUSE_OK or a negative HFUSE_ERR_* code; nothing is thrown;
 *   - calls are asynchronous with respect to the host;
 *   - thread-safe per (device, stream); the library holds no mutable state except the
 *     tuning table changed by hfuse_tune_set().
 */
#ifndef HFUSE_B200_H
#define HFUSE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define HFUSE_API __attribute__((visibility("default")))
#else
#define HFUSE_API
#endif

typedef void* hfuse_stream_t;

enum {
    HFUSE_OK = 0,
    HFUSE_ERR_BAD_ARG = -1,     /* null pointer, non-positive extent, inconsistent shape */
    HFUSE_ERR_ALIGNMENT = -2,   /* a buffer is not 16-byte aligned */
    HFUSE_ERR_TOO_LARGE = -3,   /* an extent exceeds what the kernels index */
    HFUSE_ERR_WORKSPACE = -4,   /* scratch buffer missing or too small */
    HFUSE_ERR_LAUNCH = -5,      /* cudaGetLastError() after the launch was not cudaSuccess */
    HFUSE_ERR_NO_DEVICE = -6,   /* no usable sm_100 device */
    HFUSE_ERR_UNKNOWN_PAIR = -7,
    HFUSE_ERR_NOALLOC_LIMIT = -8, /* more channels than the built-in scratch of the no-allocation entry serves */
    HFUSE_ERR_COMM = -9          /* NCCL could not be loaded, or one of its calls failed */
};

HFUSE_API const char* hfuse_error_string(int code);
HFUSE_API int hfuse_version(void);

/* ---------------------------------------------------------------------------------------
 * Parameter lists of the nine kernels, in the reference kernels' own order, as macros
 * so that a pair's prototype is literally "K1's parameters, K2's parameters".
 * P is a prefix that keeps the names of the two halves apart.
 * ------------------------------------------------------------------------------------- */

/* at::native::im2col_kernel<float>(n, im, H, W, kh, kw, ph, pw, sh, sw, dh, dw, Hc, Wc, col)
 * — configs/ml_kernels.yaml:28-36, scripts/data/ml-event.csv:17.  The reference launches it
 * once per batch item; here N and C are explicit and one launch covers the batch.
 * im [N,C,H,W] -> col [N, C*kh*kw, Hc*Wc], zero outside the image. */
#define HFUSE_IM2COL_PARAMS(P)                                                              \
    const float *P##im, int P##N, int P##C, int P##H, int P##W, int P##kh, int P##kw,       \
        int P##ph, int P##pw, int P##sh, int P##sw, int P##dh, int P##dw, float *P##col

/* at::native::MaxPoolForward<float,float>(nthreads, bottom, num, C, H, W, pH, pW, kh, kw, sh, sw,
 * ph, pw, dh, dw, top, top_mask) — configs/ml_kernels.yaml:37-45, scripts/data/ml-event.csv:5.
 * in [N,C,H,W] -> out [N,C,pH,pW] and idx (int64, h*W+w inside the plane). */
#define HFUSE_MAXPOOL_PARAMS(P)                                                             \
    const float *P##in, int P##N, int P##C, int P##H, int P##W, int P##pH, int P##pW,       \
        int P##kh, int P##kw, int P##sh, int P##sw, int P##ph, int P##pw, int P##dh,        \
        int P##dw, float *P##out, int64_t *P##idx

/* at::native::batch_norm_collect_statistics_kernel<InvStd,float,float,float,int>(input[N][C][HW],
 * eps, momentum, running_mean, running_var, save_mean, save_invstd)
 * — configs/ml_kernels.yaml:19-27, scripts/data/ml-event.csv:14.  Running statistics are
 * not touched (the reference pair passes them but the statistics kernel does not update
 * them).  `moments` is optional (may be NULL): [C][3] doubles (n, n*mean, M2 + n*mean^2),
 * the form that is summed across GPUs.  `workspace` is scratch of at least
 * hfuse_bnstats_workspace_bytes() bytes, zero-filled once by the caller before its first
 * use; each call leaves it ready for the next.  Two calls that overlap on the GPU must not
 * share a workspace. */
#define HFUSE_BNSTATS_PARAMS(P)                                                             \
    const float *P##x, int P##N, int P##C, int P##HW, float P##eps, float *P##mean,         \
        float *P##invstd, double *P##moments, void *P##workspace, size_t P##workspace_bytes

/* at::native::upsample_bilinear2d_out_frame<float,float>(n, rheight, rwidth, align_corners,
 * idata, odata) — configs/ml_kernels.yaml:1-9, scripts/data/ml-event.csv:32.  The scale
 * factors are derived from the shapes the way the operator's host side does.
 * in [N,C,H,W] -> out [N,C,outH,outW]. */
#define HFUSE_UPSAMPLE_PARAMS(P)                                                            \
    const float *P##in, int P##N, int P##C, int P##H, int P##W, int P##outH, int P##outW,   \
        int P##align_corners, float *P##out

/* at::native::kernelHistogram1D<float,float,long,1,2,-1,SHARED,Op>(a, p, b, nbins, minvalue,
 * maxvalue, totalElements, getOp) — configs/ml_kernels.yaml:10-18, scripts/data/ml-event.csv:33.
 * counts[nbins] (uint32) is cleared on the stream by the entry point, then accumulated. */
#define HFUSE_HISTC_PARAMS(P)                                                               \
    const float *P##x, int64_t P##n, int P##nbins, float P##lo, float P##hi, uint32_t *P##counts

/* ---------------------------------------------------------------------------------------
 * Standalone kernels: the unfused baseline a fused pair is compared with.
 * ------------------------------------------------------------------------------------- */
HFUSE_API int hfuse_im2col_f32(HFUSE_IM2COL_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_maxpool2d_f32(HFUSE_MAXPOOL_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_bnstats_f32(HFUSE_BNSTATS_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_upsample_bilinear2d_f32(HFUSE_UPSAMPLE_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_histc_f32(HFUSE_HISTC_PARAMS(), hfuse_stream_t stream);

HFUSE_API size_t hfuse_bnstats_workspace_bytes(int N, int C, int HW);
/* mean/invstd from moments already summed over GPUs (no counterpart in the reference,
 * which is single-GPU): mean = s1/n, var = s2/n - mean^2, invstd = 1/sqrt(var + eps). */
HFUSE_API int hfuse_bnstats_finalize_f64(const double* moments, int C, float eps, float* mean,
                                         float* invstd, hfuse_stream_t stream);

/* Batch-norm statistics without any caller-provided scratch.  It has no counterpart in the
 * reference; it exists for callers that cannot allocate device memory at the point of the
 * call (inside a framework's memory-planning phase, behind a plugin interface that passes
 * inputs and outputs only, or on a thread that must stay out of the allocator).  Same
 * arguments and results as hfuse_bnstats_f32 minus the workspace; the scratch is a static
 * device array inside the library (3,149,824 bytes on every GPU that loads it, held until
 * exit), which limits C to HFUSE_NOALLOC_MAX_CHANNELS (larger C returns
 * HFUSE_ERR_NOALLOC_LIMIT).  The call itself asks no allocator for anything.  The first call
 * on each device looks up the array's address, and with lazy module loading that is also the
 * moment the CUDA runtime loads this library's device code onto the device and the driver places
 * the array: make one warm-up call per device before any stream capture begins and before the
 * phase in which nothing may be allocated; later calls leave the device's free memory as it is.
 * All calls on a device share the one array: calls that may overlap on the GPU (different
 * streams without ordering between them) race and must be serialised by the caller. */
#define HFUSE_NOALLOC_MAX_CHANNELS 1024
HFUSE_API int hfuse_bnstats_noalloc_f32(const float* x, int N, int C, int HW, float eps, float* mean,
                                        float* invstd, double* moments, hfuse_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Fused pairs.  One kernel launch; the block is split into K1's and K2's thread ranges,
 * each synchronising only on its own named barrier.  Order of the halves follows the
 * reference's pair lists (configs/ml_fusion.yaml, line numbers beside each).
 * ------------------------------------------------------------------------------------- */
HFUSE_API int hfuse_im2col_maxpool_f32(HFUSE_IM2COL_PARAMS(a_), HFUSE_MAXPOOL_PARAMS(b_),
                                       hfuse_stream_t stream);                        /* ml_fusion.yaml:1-4   */
HFUSE_API int hfuse_im2col_bnstats_f32(HFUSE_IM2COL_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_),
                                       hfuse_stream_t stream);                        /* ml_fusion.yaml:5-8   */
HFUSE_API int hfuse_im2col_histc_f32(HFUSE_IM2COL_PARAMS(a_), HFUSE_HISTC_PARAMS(b_),
                                     hfuse_stream_t stream);                          /* ml_fusion.yaml:9-12  */
HFUSE_API int hfuse_im2col_upsample_f32(HFUSE_IM2COL_PARAMS(a_), HFUSE_UPSAMPLE_PARAMS(b_),
                                        hfuse_stream_t stream);                       /* ml_fusion.yaml:13-16 */
HFUSE_API int hfuse_maxpool_bnstats_f32(HFUSE_MAXPOOL_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_),
                                        hfuse_stream_t stream);                       /* ml_fusion.yaml:17-20 */
HFUSE_API int hfuse_maxpool_upsample_f32(HFUSE_MAXPOOL_PARAMS(a_), HFUSE_UPSAMPLE_PARAMS(b_),
                                         hfuse_stream_t stream);                      /* ml_fusion.yaml:21-24 */
HFUSE_API int hfuse_histc_maxpool_f32(HFUSE_HISTC_PARAMS(a_), HFUSE_MAXPOOL_PARAMS(b_),
                                      hfuse_stream_t stream);                         /* ml_fusion.yaml:25-28 */
HFUSE_API int hfuse_histc_upsample_f32(HFUSE_HISTC_PARAMS(a_), HFUSE_UPSAMPLE_PARAMS(b_),
                                       hfuse_stream_t stream);                        /* ml_fusion.yaml:29-32 */
HFUSE_API int hfuse_upsample_bnstats_f32(HFUSE_UPSAMPLE_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_),
                                         hfuse_stream_t stream);                      /* ml_fusion.yaml:33-36 */
HFUSE_API int hfuse_histc_bnstats_f32(HFUSE_HISTC_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_),
                                      hfuse_stream_t stream);                         /* ml_fusion.yaml:37-40 */

/* ---------------------------------------------------------------------------------------
 * Backward kernels.  The reference lists them beside the forward kernels but fuses none of
 * them (configs/ml_kernels.yaml:46-63: max_pool_backward_nchw, and batch_norm_backward_kernel,
 * its only kernel with HasBarriers: true).
 *   max-pool: grad_in[n,c,h,w] = sum of grad_out over the outputs whose index is h*W+w
 *             (idx as written by hfuse_maxpool2d_f32).
 *   batch-norm (training mode, saved mean / invstd from the statistics kernel; weight may be
 *             NULL = 1; grad_in / grad_weight / grad_bias may each be NULL):
 *             grad_bias = sum(dy), grad_weight = sum(dy (x-mean)) invstd,
 *             grad_in = (dy - sum(dy)/M - (x-mean) invstd^2 sum(dy (x-mean))/M) invstd weight.
 * The pair runs both in one block (max-pool range | batch-norm range with its named barrier).
 * ------------------------------------------------------------------------------------- */
HFUSE_API int hfuse_maxpool2d_backward_f32(const float* grad_out, const int64_t* idx, int N, int C, int H, int W,
                                           int pH, int pW, int kh, int kw, int sh, int sw, int ph, int pw, int dh,
                                           int dw, float* grad_in, hfuse_stream_t stream);
HFUSE_API int hfuse_bn_backward_f32(const float* x, const float* grad_out, int N, int C, int HW, const float* weight,
                                    const float* mean, const float* invstd, float* grad_in, float* grad_weight,
                                    float* grad_bias, hfuse_stream_t stream);
HFUSE_API int hfuse_maxpool_backward_bn_backward_f32(
    const float* p_grad_out, const int64_t* p_idx, int pN, int pC, int pHin, int pWin, int pH, int pW, int kh, int kw,
    int sh, int sw, int ph, int pw, int dh, int dw, float* p_grad_in, const float* x, const float* grad_out, int N, int C,
    int HW, const float* weight, const float* mean, const float* invstd, float* grad_in, float* grad_weight,
    float* grad_bias, hfuse_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Multi-GPU batch-norm statistics with the cross-GPU sum inside the kernel (no counterpart
 * in the reference, which is single-GPU).  One process per GPU; each creates an exchange
 * object (a small device buffer), publishes its IPC handle, collects every rank's handle
 * (any transport: torch.distributed, MPI, a file) and connects.  The *_allreduce entry
 * points then behave like their plain namesakes except that mean / invstd (and `moments`)
 * are the statistics over ALL ranks' batches: the statistics thread range stores each
 * channel's moments into every rank's buffer over NVLink and folds all ranks' rows once the
 * last one has arrived.  Rules: every rank makes the same sequence of calls on one exchange
 * object; calls on one object go to one stream; the in-kernel wait for the other ranks gives
 * up after 5 s and raises the flag hfuse_exchange_status reports (results are then invalid).
 * Which slot of the buffer a call uses is counted on the device, by the kernels themselves, so
 * the calls may be captured in a CUDA graph and replayed any number of times (every rank must
 * replay the same number of calls), and a call that returned an error never ran and does not
 * count.  The status flag stays raised until hfuse_exchange_clear_status.
 * ------------------------------------------------------------------------------------- */
#define HFUSE_IPC_HANDLE_BYTES 64
#define HFUSE_MAX_RANKS 8
typedef struct hfuse_exchange hfuse_exchange;
HFUSE_API int hfuse_exchange_create(int world, int rank, int channels, hfuse_exchange** out);
HFUSE_API int hfuse_exchange_local_handle(hfuse_exchange* ex, uint8_t handle[HFUSE_IPC_HANDLE_BYTES]);
/* handles: world x HFUSE_IPC_HANDLE_BYTES bytes in rank order (host memory); the own entry is ignored */
HFUSE_API int hfuse_exchange_connect(hfuse_exchange* ex, const uint8_t* handles);
/* One process that drives several GPUs connects without IPC: it takes every exchange object's
 * buffer (hfuse_exchange_local_pointer) and gives each object the list of all of them in rank
 * order; peer access between the devices must be enabled by the caller.  The own entry is ignored. */
HFUSE_API int hfuse_exchange_local_pointer(hfuse_exchange* ex, void** buffer);
HFUSE_API int hfuse_exchange_connect_pointers(hfuse_exchange* ex, void* const* buffers);
/* limit of the in-kernel wait for the other ranks' moments (default 5 s), for later calls */
HFUSE_API int hfuse_exchange_set_timeout(hfuse_exchange* ex, uint64_t nanoseconds);
HFUSE_API int hfuse_exchange_status(hfuse_exchange* ex, int* timed_out);   /* synchronises the device */
/* lowers the flag again, ordered after the earlier work on `stream` */
HFUSE_API int hfuse_exchange_clear_status(hfuse_exchange* ex, hfuse_stream_t stream);
HFUSE_API int hfuse_exchange_destroy(hfuse_exchange* ex);
HFUSE_API int hfuse_bnstats_allreduce_f32(HFUSE_BNSTATS_PARAMS(), hfuse_exchange* ex, hfuse_stream_t stream);
HFUSE_API int hfuse_upsample_bnstats_allreduce_f32(HFUSE_UPSAMPLE_PARAMS(a_), HFUSE_BNSTATS_PARAMS(b_),
                                                   hfuse_exchange* ex, hfuse_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Crypto nonce searches.
 *
 * Reference kernels (configs/crypto_kernels.yaml:1-32, signatures in
 * scripts/data/ethminer_event.csv:2-27):
 *   ethash_search(volatile Search_results* g_output, uint64_t start_nonce)
 *   blake2b_gpu_hash(uint32 threads, uint32 startNonce, uint32* resNonce, uint2 target2)
 *       — the kernel the reference labels "Blake256" (scripts/analyze_nvprof.py:78)
 *   sha256d_gpu_hash_shared(uint32 threads, uint32 startNonce, uint32* resNonces)
 *   sia_blake2b_gpu_hash(uint32 threads, uint32 startNonce, uint32* resNonce, uint2 target2)
 * Those kernels take header, target and DAG from __constant__ symbols; here they are
 * arguments, so concurrent calls on different streams do not interfere.
 *
 * A digest is a hit iff its 32 bytes read as a big-endian 256-bit integer are below
 * `target` (32 bytes, big-endian, host memory).  Headers are host memory.
 *   BLAKE-256 (14 rounds) / SHA-256d : 80-byte header, 32-bit little-endian nonce at bytes
 *       76..79; nonce = (uint32)(start + i), i < count <= 2^32.
 *   Sia BLAKE2b-256 : 80-byte header, 64-bit little-endian nonce at bytes 32..39.
 *   ethash : Keccak-512(header_hash[32] || nonce as 8 little-endian bytes), 64 DAG
 *       accesses of 128 bytes, mix digest and Keccak-256 result per the public
 *       specification; `dag` holds dag_items x 128 bytes on the device.
 * ------------------------------------------------------------------------------------- */
#define HFUSE_MAX_HITS 256

/* The result record (replaces the reference's `Search_results`, whose layout is in the
 * absent ethminer sources).  Device memory; reset it before every search (hfuse_hits_reset):
 * `count` must start at zero and counts every hit found even beyond HFUSE_MAX_HITS; slots
 * are filled in arrival order, so sort by nonce before comparing.  `reserved` is the work
 * queue cursor of the fused searches and of the work-queue form of the standalone ones (warps
 * take chunks of nonces from it); the entry points clear it themselves.  The two halves of a fused search need two DIFFERENT
 * records (one record for both returns HFUSE_ERR_BAD_ARG).  count <= 2^61 (2^32 for the 32-bit
 * nonces). */
typedef struct hfuse_hits {
    uint32_t count;
    uint32_t reserved;
    uint64_t nonce[HFUSE_MAX_HITS];
    uint32_t mix[HFUSE_MAX_HITS][8];   /* ethash mix digest, little-endian words; zero otherwise */
} hfuse_hits;

HFUSE_API int hfuse_hits_reset(hfuse_hits* hits, hfuse_stream_t stream);

#define HFUSE_BLAKE256_PARAMS(P)                                                            \
    const uint8_t *P##header80, uint64_t P##start, uint64_t P##count, const uint8_t *P##target32, \
        hfuse_hits *P##hits
#define HFUSE_SHA256D_PARAMS(P) HFUSE_BLAKE256_PARAMS(P)
#define HFUSE_SIA_PARAMS(P) HFUSE_BLAKE256_PARAMS(P)
#define HFUSE_ETHASH_PARAMS(P)                                                              \
    const void *P##dag, uint32_t P##dag_items, const uint8_t *P##header_hash32, uint64_t P##start, \
        uint64_t P##count, const uint8_t *P##target32, hfuse_hits *P##hits

/* Standalone searches.  Every search is compiled as a grid-stride sweep and as a work queue
 * (variants "T:0:minBlocks" and "T:0:minBlocks queue" of hfuse_tune_describe); the compiled default
 * is whichever the sweep on B200 found faster (ethash: the queue, 676 vs 581 MH/s over 2^30 nonces). */
HFUSE_API int hfuse_blake256_search(HFUSE_BLAKE256_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_sha256d_search(HFUSE_SHA256D_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_sia_blake2b_search(HFUSE_SIA_PARAMS(), hfuse_stream_t stream);
HFUSE_API int hfuse_ethash_search(HFUSE_ETHASH_PARAMS(), hfuse_stream_t stream);

/* pair order follows configs/crypto_fusion.yaml (line numbers beside each) */
HFUSE_API int hfuse_ethash_blake256_search(HFUSE_ETHASH_PARAMS(a_), HFUSE_BLAKE256_PARAMS(b_),
                                           hfuse_stream_t stream);                    /* crypto_fusion.yaml:1-4   */
HFUSE_API int hfuse_sha256d_ethash_search(HFUSE_SHA256D_PARAMS(a_), HFUSE_ETHASH_PARAMS(b_),
                                          hfuse_stream_t stream);                     /* crypto_fusion.yaml:5-8   */
HFUSE_API int hfuse_sia_ethash_search(HFUSE_SIA_PARAMS(a_), HFUSE_ETHASH_PARAMS(b_),
                                      hfuse_stream_t stream);                         /* crypto_fusion.yaml:9-12  */
HFUSE_API int hfuse_blake256_sha256d_search(HFUSE_BLAKE256_PARAMS(a_), HFUSE_SHA256D_PARAMS(b_),
                                            hfuse_stream_t stream);                   /* crypto_fusion.yaml:13-16 */
HFUSE_API int hfuse_blake256_sia_search(HFUSE_BLAKE256_PARAMS(a_), HFUSE_SIA_PARAMS(b_),
                                        hfuse_stream_t stream);                       /* crypto_fusion.yaml:17-20 */
HFUSE_API int hfuse_sha256d_sia_search(HFUSE_SHA256D_PARAMS(a_), HFUSE_SIA_PARAMS(b_),
                                       hfuse_stream_t stream);                        /* crypto_fusion.yaml:21-24 */

/* ethash DAG generation — the step before the search (reference: 16 launches of
 * ethash_calculate_dag_item ahead of every search, scripts/data/miner.json:10052).  Public
 * ethash specification: the light cache (cache_nodes x 64 bytes, host memory, sequential
 * Keccak-512 chain plus three mixing rounds) is built on the host; DAG node i (64 bytes) =
 * Keccak-512 over 256 FNV-mixed cache parents.  Nodes [first_node, first_node + node_count)
 * are written at dag + 64 * node (device); a 128-byte DAG item of the search is two nodes. */
HFUSE_API int hfuse_ethash_make_cache(const uint8_t seed32[32], uint32_t cache_nodes, void* host_cache);
HFUSE_API int hfuse_ethash_generate_dag(const void* cache, uint32_t cache_nodes, void* dag, uint32_t first_node,
                                        uint32_t node_count, hfuse_stream_t stream);

/* Single-hash device evaluation for tests: digest (and ethash mix) of `count` consecutive
 * nonces, written to out32[count][32] (and mix32[count][32], may be NULL unless kind 3).
 * kind: 0 BLAKE-256, 1 SHA-256d, 2 Sia BLAKE2b, 3 ethash (header = header_hash32). */
HFUSE_API int hfuse_hash_batch(int kind, const uint8_t* header, const void* dag, uint32_t dag_items,
                               uint64_t start, uint32_t count, uint8_t* out32, uint8_t* mix32,
                               hfuse_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Multi-GPU entry points for hosts written in C or C++ (no counterpart in the reference, which
 * is single-GPU): one process or host thread per GPU, NCCL underneath (loaded at run time from
 * libnccl.so.2; without it these calls return HFUSE_ERR_COMM and everything else still works).
 * Rank 0 makes an id (hfuse_comm_unique_id), hands it to the other ranks by any transport, and
 * every rank calls hfuse_comm_create with its own GPU current (a collective call).
 *   hfuse_bnstats_allreduce_nccl_f64: sums the [C][3] double moments that hfuse_bnstats_f32 (or a
 *       pair with it) wrote on every rank, in place, then mean / invstd of the whole batch — the
 *       library-collective counterpart of the in-kernel exchange above;
 *   hfuse_histc_allreduce_counts: sums the histogram counts of the batch shards, in place;
 *   hfuse_dag_broadcast: rank `root` sends its DAG to all others (instead of every rank
 *       generating its own copy);
 *   *_search_sharded: the fused search over this rank's contiguous share of both nonce ranges
 *       (hfuse_shard_range); hits stay in the rank's records, the host merges and sorts them.
 * ------------------------------------------------------------------------------------- */
#define HFUSE_COMM_ID_BYTES 128
typedef struct hfuse_comm hfuse_comm;
HFUSE_API int hfuse_comm_unique_id(uint8_t id[HFUSE_COMM_ID_BYTES]);
HFUSE_API int hfuse_comm_create(int world, int rank, const uint8_t id[HFUSE_COMM_ID_BYTES], hfuse_comm** out);
HFUSE_API int hfuse_comm_destroy(hfuse_comm* comm);
HFUSE_API int hfuse_bnstats_allreduce_nccl_f64(hfuse_comm* comm, double* moments, int C, float eps, float* mean,
                                               float* invstd, hfuse_stream_t stream);
HFUSE_API int hfuse_histc_allreduce_counts(hfuse_comm* comm, uint32_t* counts, int nbins, hfuse_stream_t stream);
HFUSE_API int hfuse_dag_broadcast(hfuse_comm* comm, void* dag, size_t bytes, int root, hfuse_stream_t stream);
HFUSE_API int hfuse_blake256_sha256d_search_sharded(HFUSE_BLAKE256_PARAMS(a_), HFUSE_SHA256D_PARAMS(b_), int rank,
                                                    int world, hfuse_stream_t stream);
HFUSE_API int hfuse_sia_ethash_search_sharded(HFUSE_SIA_PARAMS(a_), HFUSE_ETHASH_PARAMS(b_), int rank, int world,
                                              hfuse_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Tuning (the reference sweeps the split in 128-thread steps and a launch-bound register
 * cap per pair, tools/llvm-smart-fuser/main.cpp:182-236; here each pair has a compiled
 * list of (T1, T2, blocks/SM) variants).  `pair` is the entry point's name without the
 * "hfuse_" prefix and type suffix, e.g. "im2col_maxpool".  variant < 0 restores the
 * default.  hfuse_tune_describe writes "T1:T2:minBlocks" of a variant into buf and
 * returns the number of variants, or a negative error.
 * ------------------------------------------------------------------------------------- */
HFUSE_API int hfuse_tune_set(const char* pair, int variant, int blocks_per_sm);
HFUSE_API int hfuse_tune_describe(const char* pair, int variant, char* buf, size_t buflen);
/* Index of the compiled default variant of a kernel or pair (what runs while hfuse_tune_set has
 * not chosen another one), or HFUSE_ERR_UNKNOWN_PAIR.  "upsample_bnstats_allreduce_wide" names the
 * exchange pair's default with more than four ranks. */
HFUSE_API int hfuse_tune_default(const char* pair);
/* "upsample_bnstats_allreduce" only: per mille (0..1000, -1 = compiled default) of the upsample's
 * items that the statistics thread range takes over between sending its moments to the peers and
 * waiting for theirs.  Any other name: HFUSE_ERR_UNKNOWN_PAIR. */
HFUSE_API int hfuse_tune_set_share(const char* pair, int permille);

/* Named switches between alternative code paths of a kernel.  Unknown name: HFUSE_ERR_UNKNOWN_PAIR.
 *   "im2col_store_path": how the im2col role writes 3x3 / stride 1 / pad 1 shapes.  0 = it keeps
 *       its patch in registers and writes the taps with 256-bit streaming stores; 1 = it goes
 *       through a shared-memory tile and the taps leave as bulk (TMA) copies of whole bands of
 *       rows; -1 (the default) = whichever the sweep on B200 found faster for the kernel or pair
 *       that is called.  Same bytes either way.
 *   "bnstats_load_path": how the statistics role reads its input when one block handles a whole
 *       channel and the rows of one image (HW floats) are 1 to 25 KB long and 16-byte multiples.
 *       0 = 16-byte loads into registers; 1 = bulk (TMA) copies of whole rows into two
 *       shared-memory buffers, completion counted on an mbarrier, summed from shared memory;
 *       -1 (the default) = the compiled choice per kernel or pair.  Same statistics to rounding.
 *   "histc_load_path": how the histogram role reads its input (up to 256 bins).  0 = 16-byte loads
 *       into registers; 1 = one thread brings chunks of the input into a ring of shared-memory
 *       buffers with bulk (TMA) copies ("full" and "empty" mbarriers per buffer) and the others count
 *       out of shared memory; -1 (the default) = the compiled choice.  Same counts either way.
 *   "exchange_pair_pool": how hfuse_upsample_bnstats_allreduce_f32 divides the upsample between its
 *       two thread ranges.  1 = every warp of the block draws 32-item chunks from one cursor (the
 *       statistics range joins after it has sent its moments); 0 = a fixed share goes to the
 *       statistics range (hfuse_tune_set_share; setting a share selects this form too); -1 (the
 *       default) = the compiled choice. */
HFUSE_API int hfuse_tune_option(const char* name, int value);

/* Host utility (no counterpart in the reference, which is single-GPU): the share of `total` batch
 * items or nonces that rank `rank` of `world` works on, one process per GPU.  Contiguous and
 * balanced: the first total % world ranks get one item more; a length may be zero.  A sharded
 * nonce sweep is hfuse_*_search(start + offset, length) on every rank. */
HFUSE_API int hfuse_shard_range(uint64_t total, int rank, int world, uint64_t* offset, uint64_t* length);

/* Host utility: xoshiro256** byte stream (state = four splitmix64 outputs of `seed`,
 * little-endian u64 words) — the generator the synthetic DAG and headers are drawn from. */
HFUSE_API void hfuse_xoshiro256ss_fill(uint64_t seed, void* host_dst, size_t nbytes);

/* Measurement utility (no counterpart in the reference): one launch of a kernel that does
 * nothing but independent 32-bit add / xor / rotate chains on every SM, the operation mix of
 * the hash searches.  mix 0 = xor + rotate, 1 = add + xor + rotate on the integer pipe,
 * 2 = the same with the add issued as a multiply-add (the arrangement the hash roles use).
 * Writes the number of 32-bit lane operations the launch performs to *lane_ops (host); the
 * caller times the launch and divides.  `sink` is 4 device bytes that are never written. */
HFUSE_API int hfuse_int32_probe(int mix, uint32_t iters, uint32_t* sink, uint64_t* lane_ops, hfuse_stream_t stream);

/* Measurement utility (no counterpart in the reference): one launch that reads read_bytes from src
 * (16-byte loads) and writes write_bytes to dst (32-byte streaming stores) and does nothing else:
 * the memory-traffic mix of a kernel, without the kernel.  read_bytes / 16 <= write_bytes / 32;
 * dst 32-byte aligned, src 16-byte aligned, sizes multiples of 32 and 16. */
HFUSE_API int hfuse_hbm_probe(const void* src, size_t read_bytes, void* dst, size_t write_bytes, hfuse_stream_t stream);
/* The same traffic with the writes issued as bulk (TMA) copies of 8 KB from shared memory instead of
 * streaming stores: write_bytes a multiple of 8192, read_bytes <= write_bytes. */
HFUSE_API int hfuse_hbm_probe_bulk(const void* src, size_t read_bytes, void* dst, size_t write_bytes, hfuse_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HFUSE_B200_H */
