/* C ABI of librf_b200.so - the B200 (sm_100a) drop-in for the two hot paths of
 * RadeonFlow_Kernels: the FP8 block-scaled GEMM and the MoE layer.
 *
 * Plain pointers and sizes only.  All device pointers are CUDA device
 * addresses on the current device; all calls are stream-ordered and return
 * before the work completes unless stated otherwise.
 *
 * Each declaration cites the reference interface it replaces (path inside the
 * reference project : line).
 */
#ifndef RF_B200_H_
#define RF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (cudaStream_t). */
typedef struct CUstream_st *rf_stream_t;

/* Status codes returned by the rf_* entry points. */
enum {
    RF_OK = 0,
    RF_ERR_BAD_SHAPE = 1,      /* m,n,k violate n%64==0, k%128==0, m>0          */
    RF_ERR_NULL_POINTER = 2,
    RF_ERR_MISALIGNED = 3,     /* a, b, c must be 16-byte aligned               */
    RF_ERR_WORKSPACE = 4,      /* caller workspace too small                    */
    RF_ERR_CUDA = 5,           /* a CUDA runtime/driver call failed             */
    RF_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait expired            */
    RF_ERR_UNSUPPORTED = 7,
    RF_ERR_COMM = 8            /* collective layer reported an error            */
};

/* tests/checker/metrics.h:4-13 - same layout. */
typedef struct {
    char name[20];
    float time;   /* milliseconds */
    float gflops;
} PerfMetricEntry;

typedef struct {
    int count;
    PerfMetricEntry entries[20];
} PerfMetrics;

/* ------------------------------------------------------------------ GEMM -- */

/* Replaces `run` of src/gemm/gemm_launcher.cpp:184 (typedef in
 * tests/gemm/gemm_test.cpp:100; torch wrapper scripts/gen_submission.py:248-262).
 *
 *   C[m,n] (bf16, row-major) = sum_kb a_s[m,kb]*b_s[n/128,kb] * (A_kb . B_kb^T)
 *
 * a : e4m3 [m,k] row-major (k contiguous)     as : fp32 [m, k/128] row-major
 * b : e4m3 [n,k] row-major (k contiguous)     bs : fp32 [ceil(n/128), k/128]
 * Any m >= 1; n % 64 == 0; k % 128 == 0 (scripts/problems/gemm/task.yml:29).
 * Asynchronous on `stream`.  If `metrics` is non-NULL the call blocks until the
 * GEMM finished and fills entries[0].time / .gflops (reference: stream callback,
 * gemm_launcher.cpp:191-193).  Errors print a message and abort(), as the
 * reference does (gemm_launcher.cpp:96-100, :261-264).
 * Split-K scratch is owned by the library, per device, grown on first use.   */
void run(void *a, void *b, void *as, void *bs, void *c, int m, int n, int k, PerfMetrics *metrics,
         rf_stream_t stream);

/* Status-returning twin of `run` with caller-provided scratch.
 * `workspace` may be NULL when rf_fp8_gemm_workspace_bytes() returns 0 for the
 * shape; otherwise it must hold at least that many bytes (256-byte aligned).
 * `split_k` = 0 lets the library choose; >= 1 forces that many K slices
 * (reference: compile-time SPLITK_FACTOR, src/gemm/gemm_launcher.cpp:229-247). */
int rf_fp8_gemm(const void *a, const void *b, const float *as, const float *bs, void *c, int m, int n, int k,
                int split_k, void *workspace, size_t workspace_bytes, rf_stream_t stream);

/* Scratch bytes rf_fp8_gemm needs for this shape and split (0 = library choice).
 * Reference: init_workspace, src/gemm/gemm_launcher.cpp:30-36 (fixed 1.4 GB). */
size_t rf_fp8_gemm_workspace_bytes(int m, int n, int k, int split_k);

/* The split-K factor the library would choose for this shape on the current
 * device (reference: dispatch table, src/gemm/gemm_launcher.cpp:229-247).    */
int rf_fp8_gemm_choose_split(int m, int n, int k);

/* Reads and clears the device-side status word of the current device
 * (synchronises the device).  Returns RF_OK or RF_ERR_DEVICE_TIMEOUT; the raw
 * device code is stored in *detail when detail != NULL.
 * Reference: none - the reference aborts (include/gpu_libs.h:31-37).          */
int rf_device_status(int *detail);

/* Library / build identification: "rf_b200 <version> sm_100a".               */
const char *rf_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RF_B200_H_ */
