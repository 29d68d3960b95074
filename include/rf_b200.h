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
 * `split_k` = 0 lets the library choose; >= 1 forces that many K slices (at most 64, and at most k/128)
 * (reference: compile-time SPLITK_FACTOR, src/gemm/gemm_launcher.cpp:229-247);
 * RF_SPLIT_STREAMK (-1) asks for one pass whose ragged last wave of tiles is
 * shared out over all SMs by K blocks ("stream-K": the partial sums of a tile
 * that two or more CTAs share meet in the scratch inside the same kernel, in a
 * fixed order; no second launch).  It has no counterpart in the reference and
 * serves the same purpose as its split-K: shapes whose tile count leaves SMs
 * idle.  A shape whose tiles fill whole waves runs as a plain pass.           */
#define RF_SPLIT_STREAMK (-1)
int rf_fp8_gemm(const void *a, const void *b, const float *as, const float *bs, void *c, int m, int n, int k,
                int split_k, void *workspace, size_t workspace_bytes, rf_stream_t stream);

/* Scratch bytes rf_fp8_gemm needs for this shape and split (0 = library choice).
 * Reference: init_workspace, src/gemm/gemm_launcher.cpp:30-36 (fixed 1.4 GB). */
size_t rf_fp8_gemm_workspace_bytes(int m, int n, int k, int split_k);

/* The split-K factor the library would choose for this shape on the current
 * device (reference: dispatch table, src/gemm/gemm_launcher.cpp:229-247);
 * RF_SPLIT_STREAMK when it would run the shape as a stream-K pass.            */
int rf_fp8_gemm_choose_split(int m, int n, int k);

/* Introspection, no GPU needed: the work CTA `cta` of a launch on `num_sms` SMs goes through, in order, as
 * computed on the host by the code the kernel itself runs.  Four ints per piece: tile number, K slice, first
 * K block, end K block.  block_n 128 or 256; split_k >= 1 or RF_SPLIT_STREAMK.  Returns the number of pieces
 * (at most max_pieces are written), 0 for a CTA beyond the grid, -1 for bad arguments.                   */
int rf_fp8_gemm_work_pieces(int m, int n, int k, int block_n, int split_k, int num_sms, int cta, int *pieces,
                            int max_pieces);

/* Tuned-plan table: (tile width, split-K or RF_SPLIT_STREAMK) per exact shape, consulted before the cost model.  It replaces
 * the reference's compile-time dispatch table and the offline tuner that regenerates it
 * (src/gemm/gemm_launcher.cpp:229-247, tuner/gemm_tuner.py:343-385, tuner/gemm_batch.py:8-27).
 * block_n: 128 or 256 (tile 128 x block_n), 512 = CTA pair (256 x 256); block_n == 0 removes the entry.
 * The library starts with a built-in table for the benchmark shapes (RF_FP8_GEMM_NO_BUILTIN_PLANS=1 drops
 * it) and reads the file named by RF_FP8_GEMM_PLANS at first use.                                       */
int rf_fp8_gemm_set_plan(int m, int n, int k, int block_n, int split_k);
/* The plan the library would use (table entry or cost model; 148 SMs assumed when no GPU is present).   */
int rf_fp8_gemm_get_plan(int m, int n, int k, int *block_n, int *split_k);
/* Text file, one "m n k block_n split_k" per line, '#' comments (what `python -m
 * radeonflow_kernels_b200.tune` writes).  Returns the number of entries loaded, -1 if the file cannot be
 * read, -2 if a line was malformed (the valid lines are still loaded).                                  */
int rf_fp8_gemm_load_plans(const char *path);

/* Same arithmetic with the operands in the reference's own physical layout
 * (src/gemm/gemm_kernel_legacy.cpp:264-268; scripts/problems/gemm/reference.py:28-37 creates (k,m) and
 * returns .T): a [k][m], b [k][n] (m / n contiguous), as [k/128][m], bs [k/128][ceil(n/128)], c [m][n].
 * The tiles are consumed as MN-major tensor-core operands, so the reference's two transpose passes
 * (src/gemm/gemm_launcher.cpp:55-56, src/gemm/transpose_kernel.cpp) have no counterpart.  m % 16 == 0.
 * Bytes are still OCP e4m3fn.  workspace == NULL uses the library-owned scratch.               */
int rf_fp8_gemm_colmajor(const void *a, const void *b, const float *as, const float *bs, void *c, int m, int n,
                         int k, void *workspace, size_t workspace_bytes, rf_stream_t stream);

/* rf_fp8_gemm_colmajor for operands whose bytes are e4m3fnuz (bias 8, the MI300X format the reference
 * computes in: __hip_fp8_e4m3_fnuz, src/gemm/gemm_kernel.cpp:30-34; tests/checker/checker.cpp casts to
 * torch.float8_e4m3fnuz).  A fnuz byte read as OCP e4m3fn is exactly twice its value, subnormals included,
 * so the tensor cores consume the bytes unchanged and the epilogue folds 1/2 per operand into the scale
 * product (exact).  Three fnuz bytes have no counterpart under that reading: 0x80 (NaN), 0x7F and 0xFF
 * (+-240, which amax-scaled quantisation puts into practically every 128-block).  One pass per operand
 * ahead of the GEMM writes the e4m3fn bytes of EQUAL value into library-owned scratch (m*k + n*k bytes,
 * grown on first use) and flags an operand that holds one of the three bytes; the GEMM then reads that
 * operand from the converted copy (no 1/2 for it).  The conversion is exact except for the 15 magnitudes
 * below 2^-6, which lie between e4m3fn's subnormals and are rounded to nearest-even there (absolute
 * error <= 2^-10, i.e. <= 4e-6 of a block whose largest magnitude is 240); fnuz NaN stays NaN.  Operands
 * without special bytes are computed from the caller's bytes, exactly.  Nothing is synchronised and the
 * result is always written; rf_device_status() afterwards reports detail 16 once if a converted copy was
 * used (a note, not an error: status word 1 never stops a kernel).  m*k and n*k must be multiples of 16. */
int rf_fp8_gemm_colmajor_fnuz(const void *a, const void *b, const float *as, const float *bs, void *c, int m,
                              int n, int k, void *workspace, size_t workspace_bytes, rf_stream_t stream);

/* Allocation-free variant of rf_fp8_gemm.  It has no counterpart in the reference (whose `run`
 * allocates its scratch lazily with hipMalloc, src/gemm/gemm_launcher.cpp:30-36).
 *
 * For callers that cannot allocate device memory where the GEMM runs and cannot pass a scratch
 * pointer either: code between graph capture and replay, latency-critical threads that must not
 * enter the CUDA allocator (it can lock and implicitly synchronise the device), and embedders whose
 * GPU memory belongs to another allocator.  The split-K slices live in a fixed array inside the
 * loaded library image: RF_STATIC_SCRATCH_BYTES (16 MiB) on every GPU that loads the library, held
 * until the process exits.  No cudaMalloc/cudaFree or other allocating call is made, at set-up or
 * per call.
 *
 * Limits and rules:
 *  - An explicit split_k >= 2 needs split_k * m * n * 4 bytes to fit in RF_STATIC_SCRATCH_BYTES (and
 *    RF_SPLIT_STREAMK what rf_fp8_gemm_workspace_bytes reports for it);
 *    otherwise RF_ERR_WORKSPACE is returned and a message names the sizes.  split_k = 0 lets the
 *    library choose: when its usual plan for the shape would not fit, it runs the shape unsplit
 *    (split_k = 1 never needs scratch) instead of refusing.
 *  - The first call on each device looks up the array's device address and sets kernel attributes;
 *    make that first call before starting any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's slices.  Nothing in
 *    it needs clearing (every slice element is rewritten before it is read), but two calls that can
 *    overlap on the GPU (different streams without an ordering between them) race on it.
 *  - A bounded device-side wait that expires is recorded in a status area private to this path;
 *    rf_fp8_gemm_static_status reads and clears it.                                                */
#define RF_STATIC_SCRATCH_BYTES (16u << 20)
int rf_fp8_gemm_static_scratch(const void *a, const void *b, const float *as, const float *bs, void *c, int m,
                               int n, int k, int split_k, rf_stream_t stream);

/* rf_device_status for the allocation-free path (no counterpart in the reference): synchronises the
 * device, reads the path's own status area through the symbol's device address, clears it and returns
 * RF_OK or RF_ERR_DEVICE_TIMEOUT with the device code in *detail.  Allocates nothing.  While a code is
 * recorded, kernels of this path give up their waits early, so call it after a failure.             */
int rf_fp8_gemm_static_status(int *detail);

/* Reads and clears the device-side status area of the current device (synchronises the device).
 * Word 0 holds the code of the first bounded device-side wait that expired (1-6: producer, MMA waiting
 * for data, MMA waiting for TMEM, epilogue, scheduler / rendezvous, store); while it is set, kernels give
 * up their waits early and their output is incomplete, so callers that care check after a step.  Word 1
 * holds notes that stop nothing (16: an e4m3fnuz operand was computed from converted bytes; 32: an
 * expert-parallel receive buffer overflowed and rows were dropped).  Returns RF_OK when both are zero,
 * else RF_ERR_DEVICE_TIMEOUT with word 0 (or, if that is zero, word 1) in *detail.
 * Reference: none - the reference aborts (include/gpu_libs.h:31-37).                                 */
int rf_device_status(int *detail);

/* Limit of every bounded device-side wait on the current device, in nanoseconds (0 = the default, 2 s).
 * Stored in the status area and read by the kernels when a wait runs long; takes effect for kernels
 * launched afterwards.  No reference counterpart.                                                  */
int rf_set_wait_limit_ns(unsigned long long limit_ns);

/* ------------------------------------------------------------------- MoE -- */

/* src/moe/moe.h:3-12 */
typedef struct {
    int batch_size;
    int seq_len;
    int d_hidden;
    int d_expert;
    int n_routed_experts;
    int n_experts_per_token;
    int n_shared_experts;
    int seed;
} InputParams;

/* src/moe/moe.h:14-65 - identical field order.  Every pointer is a device
 * buffer supplied by the caller except expert_weight_{gate,up,down}, which are
 * HOST arrays of n_routed_experts device pointers (tests/moe/moe_topk_test.cpp:140-152).
 * The *_transposed and *_splitk fields are accepted and ignored.             */
typedef struct {
    InputParams params;
    void **expert_weight_gate;  /* [E] -> fp16 [d_hidden, d_expert] row-major */
    void **expert_weight_up;    /* [E] -> fp16 [d_hidden, d_expert]           */
    void **expert_weight_down;  /* [E] -> fp16 [d_expert, d_hidden]           */

    void *expert_weight_gate_transposed;
    void *expert_weight_up_transposed;
    void *expert_weight_down_transposed;

    void *input_seq;            /* fp16 [T, d_hidden], T = batch_size*seq_len */

    void *shared_expert_weight_gate; /* fp16 [d_hidden, d_expert*n_shared]    */
    void *shared_expert_weight_gate_transposed;
    void *shared_expert_weight_up;
    void *shared_expert_weight_up_transposed;
    void *shared_expert_weight_down; /* fp16 [d_expert*n_shared, d_hidden]    */
    void *shared_expert_weight_down_transposed;

    void *router_weight;        /* fp16 [E, d_hidden]                         */

    void *expert_scores;        /* fp16 [T, E] router logits (input; see run_topk) */

    void *seq_experts_index;    /* int32 [T, k]                               */
    void *seq_experts_softmax;  /* fp16  [T, k]                               */

    void *source_rows;          /* int32 [T*k], value = k_idx*T + t           */

    void *permuted_experts;     /* int32 [T*k] sorted expert ids              */
    void *permuted_rows;        /* int32 [T*k] source_rows in sorted order    */

    void *first_token_offset;   /* int32 [E+1]                                */

    void *expanded_seq_input;   /* fp16 [T*k, d_hidden]                       */
    void *expanded_seq_softmax; /* fp16 [T*k]                                 */
    void *rev_permuted_rows;    /* int32 [T*k]                                */

    void *expanded_fc1_output;  /* fp16 [T*k, d_expert]                       */
    void *expanded_fc1_gate_splitk;
    void *expanded_fc1_up_splitk;
    void *expanded_fc2_output;  /* fp16 [T*k, d_hidden]                       */
    void *expanded_fc2_splitk;

    void *shared_fc1_output;    /* fp16 [T, d_expert*n_shared]                */
    void *shared_fc1_gate_splitk;
    void *shared_fc1_up_splitk;
    void *shared_fc2_output;    /* fp16 [T, d_hidden]                         */
    void *shared_fc2_splitk;

    void *final_output;         /* fp16 [T, d_hidden]                         */
    void *final_output_splitk;
} MoEInputRaw;

/* Replaces `run_topk` of src/moe/moe.cpp:343 (typedef tests/moe/moe_topk_test.cpp:400).
 * Runs the whole layer on `stream` from the router logits in
 * input->expert_scores and fills every intermediate buffer listed above.
 * Differences from the reference, all additive: any T, any power-of-two
 * E <= 256, k <= 8 (reference: 7 compiled shapes, moe.cpp:421-435); honours the
 * caller's stream; returns non-zero (RF_ERR_*) on unsupported arguments
 * instead of printing "Failed to dispatch".  When `metrics` is non-NULL the
 * call blocks until completion and fills the reference's 12 named entries
 * (moe.cpp:350-364).                                                          */
int run_topk(MoEInputRaw *input, rf_stream_t stream, PerfMetrics *metrics);

/* Like run_topk but first computes expert_scores = input_seq . router_weight^T
 * (fp16) on the device, i.e. the router GEMM the reference leaves to PyTorch
 * (scripts/gen_submission.py:400).  `router_bias` (fp32 [E], may be NULL) is
 * added to the logits before they are rounded to fp16.                        */
int rf_moe_forward(MoEInputRaw *input, const float *router_bias, rf_stream_t stream, PerfMetrics *metrics);

/* Replaces `initialize_workspace` of src/moe/moe.cpp:443: returns a
 * process-lifetime device allocation big enough for the intermediates of the
 * largest shape seen by rf_moe_workspace_reserve (default: the reference's
 * MAX_* constants, moe.cpp:36-40).                                            */
void initialize_workspace(void **workspace);

/* Bytes of intermediates for one layer call; rf_moe_bind_workspace carves a
 * caller buffer of that size into the intermediate fields of `input`
 * (reference: pointer arithmetic in run_from_python, src/moe/moe.cpp:517-578). */
size_t rf_moe_workspace_bytes(const InputParams *params);
int rf_moe_bind_workspace(MoEInputRaw *input, void *workspace, size_t workspace_bytes);

/* Replaces `run_from_python` of src/moe/moe.cpp:481-586 (python side
 * scripts/gen_submission.py:344-350, :402).  Pointers travel as integers.
 * expert_scores == 0 makes the library compute the router GEMM itself.
 * Uses the library workspace; launches on `stream`.                           */
int rf_run_from_python(int seq_len, int batch_size, int d_hidden, int d_expert, int n_routed_experts,
                       int n_experts_per_token, int n_shared_experts, unsigned long long input_seq,
                       unsigned long long expert_scores, const unsigned long long *expert_weight_gate_p,
                       const unsigned long long *expert_weight_up_p,
                       const unsigned long long *expert_weight_down_p,
                       unsigned long long shared_expert_weight_gate, unsigned long long shared_expert_weight_up,
                       unsigned long long shared_expert_weight_down, unsigned long long router_weight,
                       unsigned long long final_output, rf_stream_t stream);

/* Stage entry points (each is one reference kernel; used by the stage tests
 * and by the expert-parallel driver).                                         */

/* topk_kernel, src/moe/moe_topk_kernel.cpp:15-150: softmax over E fp16 logits,
 * k rounds of arg-max with lowest-index tie break.                            */
int rf_moe_topk(const void *expert_scores, int n_tokens, int n_experts, int top_k, void *seq_experts_index,
                void *seq_experts_softmax, void *source_rows, rf_stream_t stream);

/* sort_experts + compute_first_token_offset + the index half of expand_input
 * (src/moe/moe.cpp:119-126, src/moe/moe_topk_kernel.cpp:152-213): stable
 * counting sort of (expert, source_row) pairs.  `scratch` needs
 * rf_moe_permute_scratch_bytes(n_tokens*top_k, n_experts) bytes.                             */
size_t rf_moe_permute_scratch_bytes(int n_items, int n_experts);
int rf_moe_permute(const void *seq_experts_index, const void *source_rows, const void *seq_experts_softmax,
                   int n_tokens, int n_experts, int top_k, void *permuted_experts, void *permuted_rows,
                   void *first_token_offset, void *rev_permuted_rows, void *expanded_seq_softmax, void *scratch,
                   rf_stream_t stream);

/* expand_input row gather, src/moe/moe_topk_kernel.cpp:174-213.               */
int rf_moe_gather_rows(const void *input_seq, const void *permuted_rows, int n_tokens, int n_rows, int d_hidden,
                       void *expanded_seq_input, rf_stream_t stream);

/* Grouped expert GEMM over the row ranges group_offsets_dev[g]..[g+1] of x [n_rows, k_dim] fp16
 * (LaunchGroupGEMM, src/moe/gemm_thirdparty.cpp:65-115; one group = LaunchGEMM, :261-288).
 * `w_ptrs_host` is a HOST array of n_groups device pointers to fp16 [k_dim, n_dim] row-major
 * weights, as in MoEInputRaw.  With `w2_ptrs_host` != NULL the kernel computes
 * fp16(SiLU(fp16(X.W)) * fp16(X.W2)), the fused form of the two GEMMs plus moe_gemm_reduce_ab
 * (src/moe/moe_gemm_pipeline_kernel.cpp:51, :377-405).  n_dim % 64 == 0, k_dim % 64 == 0.
 * Row counts stay on the device (the reference copies them to the host, src/moe/moe.cpp:204). */
int rf_moe_grouped_gemm(const void *x, int n_rows, const void *const *w_ptrs_host,
                        const void *const *w2_ptrs_host, const int *group_offsets_dev, int n_groups, int n_dim,
                        int k_dim, void *out, rf_stream_t stream);

/* The grouped GEMM addresses each expert's weight through a TMA descriptor; the device arrays of
 * descriptors are cached per set of weight pointers (2048 sets by default, least recently used evicted,
 * freed only after the kernels that may read them have finished).  A set is built at a layer's first
 * call (one cudaMalloc and one blocking copy), so keep warm-up calls outside stream capture.  The MoE
 * entry points of one device share that cache and one tile-list scratch: issue them on one stream at a
 * time, as the reference does (src/moe/moe.cpp:580-583).  max_sets >= 4.  No reference counterpart
 * (hipBLASLt takes raw pointers, src/moe/gemm_thirdparty.cpp:65-115).                               */
int rf_moe_set_map_cache_sets(int max_sets);

/* on != 0: rf_moe_forward and rf_run_from_python let the first expert GEMM gather the token rows in its
 * own loader (expand_input, src/moe/moe_topk_kernel.cpp:174-213, fused) and leave expanded_seq_input
 * unwritten; run_topk always writes it, as the reference's checker expects.  Same bits either way.  Off by
 * default (RF_MOE_FUSED_GATHER=1 turns it on at first use): measured, the separate gather pass is faster.  */
int rf_moe_set_fused_gather(int on);

/* Grid cap of the grouped GEMMs that THIS host thread enqueues from now on (0 = one persistent CTA per SM,
 * the default).  The expert-parallel layer uses it to leave SMs to its dispatch kernel while the shared
 * expert runs.  No reference counterpart.                                                             */
int rf_moe_set_grid_limit(int max_ctas);

/* Router logits expert_scores[t, e] = fp16(x[t,:] . router_weight[e,:] + router_bias[e]); the
 * matmul the reference leaves to PyTorch (scripts/gen_submission.py:400).  router_bias may be NULL. */
int rf_moe_router_gemm(const void *x, const void *router_weight, const float *router_bias, int n_tokens,
                       int n_experts, int d_hidden, void *expert_scores, rf_stream_t stream);

/* reduce_output, src/moe/moe_topk_kernel.cpp:215-251.                         */
int rf_moe_combine(const void *expanded_fc2_output, const void *shared_fc2_output, const void *rev_permuted_rows,
                   const void *expanded_seq_softmax, int n_tokens, int top_k, int d_hidden, void *final_output,
                   rf_stream_t stream);

/* ------------------------------------------------------- multi-GPU (one node) -- */
/* None of these has a counterpart in the reference, which is single-GPU and has no collective
 * call (grep for nccl|rccl|mpi under src/ is empty).  One process per GPU; buffers that peers
 * touch are exported with CUDA IPC and addressed directly over NVLink.                        */

/* cudaMalloc + cudaIpcGetMemHandle: a buffer other GPUs of the node may read and write.
 * `handle64` receives the 64-byte IPC handle to send to the peers.                          */
int rf_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
/* Maps a peer's buffer into this process (enables peer access on first use).                */
int rf_peer_open(const unsigned char *handle64, void **ptr);
int rf_peer_close(void *ptr);
int rf_peer_free(void *ptr);

/* N-split FP8 GEMM with the all-gather of C fused into the epilogue: this rank owns rows
 * [rank*n/world, (rank+1)*n/world) of B and of its 128x128 scale blocks, computes that column
 * slab of C and TMA-stores every tile into the full row-major C [m, n_total] of EVERY rank
 * (`c_all[r]` = rank r's C as mapped in this process; c_all[rank] is local).  A and its scales
 * are replicated.  n_total/world must be a multiple of 128.  Completion on all ranks needs a
 * cross-rank barrier after the call (stream-ordered, e.g. a one-element NCCL all-reduce).     */
int rf_fp8_gemm_nsplit(const void *a, const void *b_shard, const float *as, const float *bs_shard,
                       void *const *c_all, int m, int n_total, int k, int rank, int world, rf_stream_t stream);

/* out[r, :] = fp16(out[r, :] + add[r, :]) for fp16 [n_rows, d_hidden] (the "+ shared[t]" of
 * reduce_output, src/moe/moe_topk_kernel.cpp:249, as a separate pass).                         */
int rf_moe_add_rows(void *out, const void *add, int n_rows, int d_hidden, rf_stream_t stream);

/* Rendezvous of the ranks of one node through peer memory, stream-ordered: every rank raises its flag
 * (the monotonically increasing `epoch` >= 1) in every peer's sync area and waits, for at most two
 * seconds, until all peers have raised theirs; work queued before it on any rank (peer stores
 * included) is complete before work queued after it on every rank.  With counts_dev != NULL the
 * n_counts int32 values are first all-gathered into row `rank` of every peer's gather area.
 * sync_all[r] = rank r's sync area as mapped here: int32 [8 + world * n_counts], zero before epoch 1;
 * the gathered matrix starts at word 8.  A wait that expires sets the device status word
 * (rf_device_status) and the kernel returns.  One launch per rank, each rank on its own GPU.     */
int rf_moe_ep_rendezvous(void *const *sync_all, const int *counts_dev, int n_counts, int rank, int world,
                         int epoch, rf_stream_t stream);

/* Expert-parallel layout: from the all-gathered pair counts counts_all_dev [world][n_experts]
 * computes, on the device, where this rank's rows land in the owners' receive buffers
 * (send_base_dev [n_experts]) and the row ranges of this rank's own experts
 * (recv_offsets_dev [n_experts/world + 1]).  Expert e lives on rank e / (n_experts/world).
 * `capacity` = rows of the receive buffers: row ranges are clipped to it and an overflow is noted in
 * the device status area (detail 32).                                                         */
int rf_moe_ep_layout(const int *counts_all_dev, int rank, int world, int n_experts, int capacity,
                     int *send_base_dev, int *recv_offsets_dev, rf_stream_t stream);

/* Dispatch: the token-row gather of expand_input (src/moe/moe_topk_kernel.cpp:174-213) writing
 * directly into the owner ranks' receive buffers `recv_x_all[r]` (fp16 [capacity, d_hidden]).
 * pair_rank / pair_row [n_pairs] record the destination of every locally sorted pair.  Rank r
 * sends to rank r+1 first, then r+2, ... so the senders never all target one GPU.
 * recv_meta_all (may be NULL): every rank's int32 [capacity] return-address table; beside row i of
 * recv_x_all[q] the sender writes recv_meta_all[q][i] = (rank << 28) | p, p = position of the pair in
 * the sender's expert-sorted order - the row_dest_dev input of rf_moe_grouped_gemm_scatter.
 * A pair whose destination row is >= capacity is NOT sent (nothing is ever written past a peer's
 * allocation): pair_rank = -1, status detail 32, and with drop_fill != NULL (this rank's fp16
 * [n_pairs, d_hidden] result rows, push variant) the pair's result row is zeroed instead.          */
int rf_moe_ep_dispatch(const void *x, const int *permuted_experts, const int *permuted_rows,
                       const int *first_token_offset, const int *send_base, int n_tokens, int n_pairs, int d_hidden,
                       int n_experts, int rank, int world, int capacity, void *const *recv_x_all,
                       void *const *recv_meta_all, int *pair_rank, int *pair_row, void *drop_fill,
                       rf_stream_t stream);

/* The experts' second GEMM fused with the way back (no reference counterpart: the reference is single-GPU;
 * it is the grouped fc2 of src/moe/moe.cpp:244-248 whose epilogue performs the row scatter that
 * reduce_output's gather, src/moe/moe_topk_kernel.cpp:215-251, would otherwise do over NVLink).
 * out row i = x[i,:] . w[group(i)] is stored, by peer stores from the GEMM's epilogue, to row
 * (row_dest_dev[i] & 0x0FFFFFFF) of dest_all[row_dest_dev[i] >> 28] (fp16 [*, n_dim]).  After a
 * rendezvous every rank holds its own pairs' expert outputs in expert-sorted order and finishes with the
 * local rf_moe_combine.                                                                          */
int rf_moe_grouped_gemm_scatter(const void *x, int n_rows, const void *const *w_ptrs_host,
                                const int *group_offsets_dev, int n_groups, int n_dim, int k_dim,
                                const int *row_dest_dev, void *const *dest_all, int world, rf_stream_t stream);

/* Combine: reduce_output (src/moe/moe_topk_kernel.cpp:215-251) reading each expert output row
 * from its owner rank's `y_all[r]` (fp16 [capacity, d_hidden]) over NVLink.  shared_fc2_output
 * may be NULL: the shared expert's rows are then added afterwards with rf_moe_add_rows, which
 * lets its second GEMM run while the combine is pulling rows over NVLink.                     */
int rf_moe_ep_combine(void *const *y_all, const void *shared_fc2_output, const int *rev_permuted_rows,
                      const void *expanded_seq_softmax, const int *pair_rank, const int *pair_row, int n_tokens,
                      int top_k, int d_hidden, int world, void *final_output, rf_stream_t stream);

/* The expert-parallel layer as one object (no reference counterpart; the host-side sequencing is the
 * multi-GPU form of run_topk_impl, src/moe/moe.cpp:129-339).  One object per rank, created with that
 * rank's device current.  It owns every buffer of a step, a side stream, the events and the rendezvous
 * epochs; rf_moe_ep_forward enqueues one whole step (router GEMM, top-k, sort, count exchange, dispatch
 * beside the shared expert, routed experts, results home, combine) without host synchronisation,
 * allocation or collective-library call.  Set-up: create on every rank -> rf_moe_ep_handles -> exchange
 * the handle blobs between the processes (any transport) -> rf_moe_ep_connect -> a barrier between the
 * processes -> forward.  Tear-down: barrier -> rf_moe_ep_disconnect on every rank -> barrier -> destroy. */
typedef struct RfMoeEp RfMoeEp;
typedef struct {
    int n_tokens;              /* tokens of THIS rank                                              */
    int d_hidden, d_expert, n_routed_experts, n_experts_per_token, n_shared_experts;
    int rank, world;           /* expert e lives on rank e / (n_routed_experts / world)            */
    int capacity;              /* rows of the receive buffers; 0 = worst case n_tokens*k*world     */
    int push_results;          /* 1: fc2's epilogue stores the results home; 0: the combine pulls  */
} RfMoeEpConfig;
#define RF_MOE_EP_HANDLE_BYTES 256   /* four 64-byte IPC handles per rank */
int rf_moe_ep_create(const RfMoeEpConfig *config, RfMoeEp **out);
/* handles: RF_MOE_EP_HANDLE_BYTES of this rank; all_handles: world blobs in rank order.        */
int rf_moe_ep_handles(RfMoeEp *ep, unsigned char *handles);
int rf_moe_ep_connect(RfMoeEp *ep, const unsigned char *all_handles);
/* Device pointers, kept by reference: router [E, d] fp16 (+ optional fp32 bias [E]); HOST arrays of the
 * n_routed_experts/world LOCAL experts' gate / up [d, f] and down [f, d]; the shared expert's three.    */
int rf_moe_ep_set_weights(RfMoeEp *ep, const void *router_weight, const float *router_bias,
                          const void *const *expert_gate, const void *const *expert_up,
                          const void *const *expert_down, const void *shared_gate, const void *shared_up,
                          const void *shared_down);
/* x: fp16 [n_tokens, d_hidden] local tokens -> out fp16 [n_tokens, d_hidden]; asynchronous on `stream`. */
int rf_moe_ep_forward(RfMoeEp *ep, const void *x, void *out, rf_stream_t stream);
enum { RF_MOE_EP_OPT_TRACE = 1,            /* value != 0: record an event after every stage of forward   */
       RF_MOE_EP_OPT_DISPATCH_BLOCKS = 2   /* value = R in 1..64: the dispatch runs as R blocks that each own
                                              an SM and move the rows with bulk copies (local HBM -> shared
                                              memory -> the owner's receive buffer), the shared expert's GEMMs
                                              on the other SMs beside them; 0: dispatch blocks on every SM, the
                                              two in turn.  Default: 32 on 2 to 4 GPUs, else 0.             */ };
int rf_moe_ep_set_option(RfMoeEp *ep, int option, int value);
/* Milliseconds of the stages of the last traced forward (synchronises); returns the number of stages.  */
int rf_moe_ep_stage_times(RfMoeEp *ep, float *ms, const char **names, int max_stages);
/* Device buffers of the last step, for tests: router logits fp16 [T, E]; top-k indices int32 [T, k]; the
 * all-gathered counts int32 [world, E]; send_base int32 [E]; recv_offsets int32 [E/world + 1]; pair_rank. */
enum { RF_MOE_EP_BUF_SCORES = 0, RF_MOE_EP_BUF_INDEX = 1, RF_MOE_EP_BUF_COUNTS_ALL = 2,
       RF_MOE_EP_BUF_SEND_BASE = 3, RF_MOE_EP_BUF_RECV_OFFSETS = 4, RF_MOE_EP_BUF_PAIR_RANK = 5 };
int rf_moe_ep_buffer(RfMoeEp *ep, int which, void **ptr, size_t *bytes);
int rf_moe_ep_disconnect(RfMoeEp *ep);
int rf_moe_ep_destroy(RfMoeEp *ep);

/* Library / build identification: "rf_b200 <version> sm_100a".               */
const char *rf_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RF_B200_H_ */
