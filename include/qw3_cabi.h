/*
 * C ABI of the B200 (sm_100a) AWQ W4A16 decode path.
 *
 * The reference (one translation unit, Inference.cu) has no FFI layer: its boundary is the C++
 * class QWen3AWQInfer (Inference.cu:356-415).  This header is what a binding of that class, or
 * of its per-operator steps, links against; include/qwen3_awq_infer.h rebuilds the class on top.
 * Every entry point returns a status (0 = QW3_OK) and never exits the process, where the
 * reference prints and calls std::exit(1) (Inference.cu:52-71).
 *
 * Conventions: pointers named d_* are device pointers on the current device; `stream` is a
 * cudaStream_t passed as void*; fp16 buffers are IEEE binary16, little endian; `pos_dev`
 * (device int32) overrides the immediate `pos` when it is not NULL, so that one captured
 * launch sequence can be replayed for every token.
 */
#ifndef QW3_CABI_H
#define QW3_CABI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum Qw3Status {
    QW3_OK = 0,
    QW3_ERR_ARG = 1,       /* bad argument / unsupported shape */
    QW3_ERR_CUDA = 2,      /* a CUDA runtime or driver call failed (see qw3_last_error) */
    QW3_ERR_IO = 3,        /* weight file missing or shorter than required (Inference.cu:299-308) */
    QW3_ERR_RANGE = 4,     /* prompt + new tokens exceed the KV capacity, token id out of range */
    QW3_ERR_TIMEOUT = 5,   /* a bounded device-side wait gave up (stage hand-off, TMA barrier) */
    QW3_ERR_DEVICE = 6,    /* not enough GPUs, or peer access unavailable (Inference.cu:566-578) */
    QW3_ERR_NOMEM = 7,
    QW3_ERR_STATE = 8      /* call not valid in the handle's current state */
};

const char* qw3_strerror(int status);
/* Message of the last failing call on this thread ("" if none). */
const char* qw3_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Operators
 * ---------------------------------------------------------------------------------------- */

/* Bit-exact materialising dequantisation; replaces dequantAwqKernel (Inference.cu:76-106) and is
 * used as a test hook only: the product path never expands the weights.
 * out[r*cols+c] = hmul(hsub(half(q), zp[g]), scale[g]), g = (c/128) mod n_groups_alloc. */
int qw3_dequant_w4(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_groups_alloc,
                   int64_t rows, int64_t cols, void* d_out_f16, void* stream);

/* Descriptor of one quantised matrix; replaces struct AWQWeight (Inference.cu:318-325) without
 * its fp16 copy d_dq.  The packed bytes stay in the on-disk layout ([out_dim][in_dim/2], low
 * nibble first).  The contraction reads them as cuBLAS reads d_dq in the reference: column-major
 * out_dim x in_dim with lda = out_dim (Inference.cu:1052-1065).  out_dim and in_dim must be
 * multiples of 128.  d_zp must be host-inspectable at creation only through `zp_integral`:
 * pass 1 when every zero-point is an integer with |zp| <= 1023 (the usual AWQ case, enables the
 * shorter exact unpack), 0 for arbitrary fp16 zero-points.  Holds no device allocation. */
typedef struct qw3_w4* qw3_w4_t;
int qw3_w4_create(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_groups_alloc,
                  int64_t out_dim, int64_t in_dim, int zp_integral, qw3_w4_t* out);
int qw3_w4_destroy(qw3_w4_t w);

/* Scratch memory of the split-K fix-up, the attention partials and the arg-max partials, plus
 * the device error word.  One workspace serves one stream: launches that share a workspace and
 * overlap on the GPU race. */
typedef struct qw3_ws* qw3_ws_t;
int qw3_ws_create(qw3_ws_t* out);
int qw3_ws_destroy(qw3_ws_t ws);
/* enable != 0: the kernels launched with this workspace use programmatic dependent launch, so that
 * a kernel's weight prefetch overlaps the tail of the kernel before it in the stream. */
int qw3_ws_set_pdl(qw3_ws_t ws, int enable);
/* Reads (and clears) the device error word: QW3_OK or QW3_ERR_TIMEOUT.  Synchronises `stream`. */
int qw3_ws_check(qw3_ws_t ws, void* stream);

enum Qw3Epilogue {
    QW3_EPI_STORE = 0,    /* y = half(acc)                                  (Inference.cu:1062)      */
    QW3_EPI_RESIDUAL = 1, /* y = hadd(y, half(acc))                         (Inference.cu:1149-1155) */
    QW3_EPI_GELU = 2,     /* y = half(gelu(half(acc)))                      (Inference.cu:271-279)   */
    QW3_EPI_ROPE_KV = 3,  /* q -> y (rotated), k (rotated), v -> cache row  (Inference.cu:1070-1103) */
    QW3_EPI_ARGMAX = 4    /* fp16 logits, first-max arg-max                 (Inference.cu:1278-1290) */
};

typedef struct Qw3GemvArgs {
    const void* d_x;        /* fp16 [in_dim] */
    const void* d_gamma;    /* fp16 [in_dim] or NULL; when set x is RMS-normalised first
                               (rmsNormKernel, Inference.cu:111-145) */
    float       eps;
    int32_t     epilogue;   /* enum Qw3Epilogue */
    void*       d_y;        /* STORE/GELU: fp16 [out_dim]; RESIDUAL: fp16 [out_dim] in/out;
                               ROPE_KV: fp16 q [out_dim/3]; ARGMAX: fp16 logits [out_dim] or NULL */
    /* ROPE_KV only: caches are [heads][max_pos][head_dim] fp16 (Inference.cu:404-407), tables are
       [max_pos][head_dim/2] fp16 (Inference.cu:444-454). */
    void*       d_k_cache;
    void*       d_v_cache;
    const void* d_cos;
    const void* d_sin;
    int32_t     heads;
    int32_t     head_dim;   /* must be 128 */
    int64_t     max_pos;
    const int32_t* d_pos;   /* device position, or NULL to use `pos` */
    int32_t     pos;
    /* ARGMAX only */
    int32_t*    d_token;    /* device int32: winning index */
    float*      d_logits_f32; /* optional fp32 copy of the fp16 logits (finalSoftmaxKernel, Inference.cu:284-292) */
} Qw3GemvArgs;

/* Fused dequantise + matrix-vector product for one token; replaces dequantAwqKernel + cublasGemmEx
 * at n = 1 (Inference.cu:1052, 1128, 1176, 1201, 1260) and the kernels the epilogue names. */
int qw3_gemv_w4a16(qw3_w4_t w, const Qw3GemvArgs* args, qw3_ws_t ws, void* stream);

/* The same product, y = half(sum_j W[i + j*out_dim] * x[j]), for callers that may not allocate: a
 * server that carved up all device memory at start-up, or a plug-in running inside another
 * framework's step, where cudaMalloc would stall the whole device.  It takes no workspace and no
 * descriptor: the split-K scratch is a fixed array inside the library (about 1.06 MiB, held by every
 * GPU that loads the library until the process exits) and the matrix is given by plain arguments.
 * It has no counterpart in the reference, which allocates everything in its constructor.
 * Limits and rules:
 *   - out_dim and in_dim are multiples of 128 and at most 16384 each; larger sizes are refused with
 *     QW3_ERR_ARG (use qw3_gemv_w4a16 with a workspace instead);
 *   - the first call on a device looks up the device address of the array and opts the kernel in to
 *     its shared-memory size; make that first call before any stream capture;
 *   - all calls on a GPU share the one array, so two calls that can overlap on that GPU (different
 *     streams) race; calls ordered on one stream are safe, and each call clears the counters it
 *     needs itself;
 *   - no cudaMalloc, cudaFree or other allocating routine is called.
 * zp_integral as in qw3_w4_create. */
int qw3_gemv_w4a16_noalloc(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_groups_alloc,
                           int64_t out_dim, int64_t in_dim, int zp_integral, const void* d_x, void* d_y,
                           void* stream);
/* Companion of qw3_gemv_w4a16_noalloc (what qw3_ws_check is to a workspace): every wait inside the kernel is bounded,
 * and one that gives up records a code in an error word of the fixed scratch instead of hanging the GPU; the call that
 * launched the kernel has returned QW3_OK long before.  This reads and clears that word on the current device:
 * QW3_ERR_TIMEOUT if a call since the last check gave up (its d_y is then void), QW3_OK otherwise.  Synchronises
 * `stream`; allocates nothing either.  qw3_gemv_w4a16_noalloc itself never clears the word. */
int qw3_gemv_w4a16_noalloc_status(void* stream);

/* Tensor-core W4A16 contraction for `rows` activations (prefill / batched rows): Y[r][i] =
 * sum_j W[i + j*out_dim] * X[r][j], fp16 in, fp32 accumulate, fp16 out.  The reference has no
 * batched path; row r of Y equals qw3_gemv_w4a16 on row r of X within fp32 summation order.
 * X is [rows][in_dim], Y is [rows][out_dim]. */
int qw3_gemm_w4a16(qw3_w4_t w, const void* d_x, int64_t rows, void* d_y, qw3_ws_t ws, void* stream);

/* rmsNormKernel (Inference.cu:111-145), standalone. */
int qw3_rmsnorm(const void* d_x, const void* d_gamma, int64_t n, float eps, void* d_out, void* stream);

/* applyRotaryKernel on q and k plus the QKV split and the KV append (Inference.cu:1070-1103) for
 * an fp16 [3*heads*head_dim] vector, standalone. */
int qw3_rope_kv_append(const void* d_qkv, void* d_q_out, void* d_k_cache, void* d_v_cache,
                       const void* d_cos, const void* d_sin, int32_t heads, int32_t head_dim,
                       int64_t max_pos, const int32_t* d_pos, int32_t pos, void* stream);

/* Decode attention for one token over cache rows 0..pos (attentionKernel, Inference.cu:182-266,
 * intended math: fp32 q.k/sqrt(d), softmax, fp32 p.v, fp16 out). */
int qw3_attn_decode(const void* d_q, const void* d_k_cache, const void* d_v_cache, int32_t heads,
                    int32_t head_dim, int64_t max_pos, const int32_t* d_pos, int32_t pos,
                    void* d_ctx, qw3_ws_t ws, void* stream);

/* The same attention for a block of `rows` consecutive prompt positions pos0 .. pos0 + rows - 1 (the batched prompt phase;
 * the reference runs attentionKernel once per prompt token, Inference.cu:1304-1343): row r of d_qkv ([rows][3 * heads * 128]
 * fp16, q in the first third, after RoPE) attends cache rows 0 .. pos0 + r, which must already hold the block's own k / v
 * rows; d_ctx is [rows][heads * 128] fp16.  From 16 rows on a tiled tensor-core kernel runs (64 query rows share each tile
 * of 64 cache rows), below that one CTA per row. */
int qw3_attn_prefill(const void* d_qkv, const void* d_k_cache, const void* d_v_cache, int32_t heads, int32_t head_dim,
                     int64_t max_pos, int32_t pos0, int32_t rows, void* d_ctx, void* stream);

/* Embedding column gather straight from the packed [hidden][vocab] matrix (gather lambda,
 * Inference.cu:1310-1315).  Token from *d_token when it is not NULL, else `token`. */
int qw3_embed_gather_w4(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_groups_alloc,
                        int64_t hidden, int64_t vocab, const int32_t* d_token, int32_t token,
                        void* d_out_f16, void* stream);

/* First-max arg-max over fp16 logits (host loop at Inference.cu:1282-1289), on the device. */
int qw3_argmax_f16(const void* d_logits, int64_t n, int32_t* d_token, qw3_ws_t ws, void* stream);

/* ------------------------------------------------------------------------------------------
 * Engine: QWen3AWQInfer behind a C handle
 * ---------------------------------------------------------------------------------------- */

#define QW3_MAX_STAGES 8

typedef struct Qw3Config {
    int32_t hidden;        /* Inference.cu:33  */
    int32_t inter;         /* Inference.cu:34  */
    int32_t heads;         /* Inference.cu:35  */
    int32_t head_dim;      /* Inference.cu:36 (128 only) */
    int32_t layers;        /* Inference.cu:37  */
    int32_t vocab;         /* Inference.cu:38  */
    int32_t max_pos;       /* Inference.cu:39: KV rows per head and RoPE table rows */
    float   eps;           /* Inference.cu:41  */
    float   rope_base;     /* Inference.cu:449 */
    int32_t sample_first;  /* 0 = reference flow (Inference.cu:1355-1363) */
    /* Layer pipeline (Inference.cu:43-47, 376-378), generalised to 1..8 stages.  Stage s runs
       layers [first_layer[s], first_layer[s+1]); all zero = even split with the remainder on the
       leading stages (8 stages of 36 layers: 5,5,5,5,4,4,4,4). */
    int32_t n_stages;
    int32_t first_layer[QW3_MAX_STAGES + 1];
    int32_t device[QW3_MAX_STAGES];  /* CUDA device of each stage; several stages may share one */
    /* One process per GPU: world > 1 makes this handle own stage `rank` only; the peers are
       connected with qw3_stage_export / qw3_stage_connect. */
    int32_t rank;
    int32_t world;
    int32_t use_graph;     /* replay one captured decode step per token */
    int32_t use_pdl;       /* programmatic dependent launch between the step's kernels */
    int32_t keep_logits;   /* keep an fp32 copy of the last step's logits (test hook) */
    int32_t persistent;    /* 2 (default): a token pass of a stage is one launch of the fused kernel (operators of a layer
                              paired, weights repacked at load time; falls back to 1 for shapes it does not cover);
                              1: one persistent kernel walking an operator list; 0: one launch per operator */
    int32_t tensor_parallel; /* with world > 1: 1 = every matrix row-split over the `world` GPUs instead of the layer pipeline (see
                                qw3_tp_export); needs n_stages = 1, device[0] = this process's GPU, persistent = 2 */
    int32_t attn_split_min;  /* fused pass: contexts longer than this many positions are split over the CTAs that share a head
                                (an exchange between them merges the parts); shorter ones are run whole by each of them.
                                0 = default (32; measured at 133, 517 and 1029 positions the split is the faster form) */
    int32_t cluster;         /* fused pass on one GPU: 1 = the CTAs that share a head form a thread-block cluster and exchange
                                through distributed shared memory (when the device can hold the clusters; 1.4 % faster on
                                the full model); 0 (default) = they exchange through global memory as they do when the
                                matrices are row-split over GPUs.  Off by default because a process that launches the
                                cooperative cluster form under Nsight Compute is terminated by the tool */
} Qw3Config;

typedef struct qw3_engine* qw3_handle;

/* Reference constants (Inference.cu:33-47) on one stage / device 0, graph and PDL on. */
int qw3_config_default(Qw3Config* cfg);

/* Constructor (Inference.cu:422-470): reads the raw .bin set named as in Inference.cu:780-900
 * from weight_dir, uploads it, zeroes the KV caches, builds the RoPE tables. */
int qw3_create(const char* weight_dir, const Qw3Config* cfg, qw3_handle* out);
int qw3_destroy(qw3_handle h);

/* generateResponse (Inference.cu:1297-1408): writes exactly max_new ids to out_ids. */
int qw3_generate(qw3_handle h, const int32_t* prompt, int32_t n_prompt, int32_t max_new,
                 int32_t* out_ids, int32_t* n_out);

/* Continues the decode loop of the last qw3_generate call for max_new more ids (same KV state,
 * positions carry on).  No counterpart in the reference, whose object is single-shot; it lets a
 * caller stream a long generation in pieces and lets a benchmark time decode steps alone. */
int qw3_decode_more(qw3_handle h, int32_t max_new, int32_t* out_ids, int32_t* n_out);

/* Prompt phase in blocks of up to 2048 rows (on = 1) instead of token by token (on = 0, the reference's flow,
 * Inference.cu:1304-1343); on = -1 (the default of a new handle) takes the blocks for prompts of 16 tokens or more and the
 * token loop below that.  In a block the four projections of a layer become the tensor-core contraction of
 * qw3_gemm_w4a16, with row versions of RMSNorm, RoPE + KV append, causal attention (tiled, on the tensor cores),
 * residual add and GeLU around them.  Per-element arithmetic is unchanged; the contractions sum in a different fp32
 * order, so cache rows and the hidden state can differ from the token loop in the last fp16 bit (the golden ids are
 * reproduced either way).  With one process per GPU (world > 1) the blocks travel from stage to stage through the
 * mailboxes' block inboxes (a peer copy between two flag kernels) and the stages overlap on successive blocks; every
 * stage must be set alike. */
int qw3_set_batched_prefill(qw3_handle h, int on);

/* One process per GPU (world > 1): from the second decode step on the stages are chained inside the token-pass
 * kernels: the last operator of a stage stores the hidden state as tagged words into the next GPU's mailbox over
 * NVLink, the first operator of the next stage polls it, and the sampled id returns to the first stage the same
 * way, so no hand-off launch sits between two stages (the reference: cudaMemcpyPeerAsync plus a host
 * synchronisation per boundary, Inference.cu:1013-1023).  on = 1 is the default; on = 0 keeps the mailbox
 * send / receive launches for every step.  Results are identical.  Every stage must be set alike. */
int qw3_set_chained_decode(qw3_handle h, int on);

/* fp32 logits of the last decode step (keep_logits = 1), vocab floats to host memory. */
int qw3_last_logits(qw3_handle h, float* out_vocab);
/* Device time of the last call's prompt loop and decode loop (CUDA events, milliseconds). */
int qw3_last_timing(qw3_handle h, float* prompt_ms, float* decode_ms);
/* Kernels launched (graph nodes included) by the last qw3_generate call. */
int qw3_last_launches(qw3_handle h, int64_t* n);

/* Test hooks for the one-layer configuration: upload KV rows [0, upto) of one layer from host
 * memory laid out [heads][upto][head_dim]; run runOneLayer (Inference.cu:1029-1230) for one token
 * with host hidden state in/out. */
int qw3_kv_upload(qw3_handle h, int32_t layer, int32_t which, const void* host_f16, int64_t upto);
int qw3_layer_decode(qw3_handle h, int32_t layer, int32_t pos, void* host_hidden_f16);

/* Test hook: the hidden state (fp16 [hidden], to host memory) that stage `stage` of this process holds after its last
 * pass, i.e. the residual stream after the stage's last layer.  With a stage split placed at the layers of interest this
 * exposes intermediate hidden states without any extra kernel. */
int qw3_stage_hidden(qw3_handle h, int32_t stage, void* host_hidden_f16);

#ifdef QW3_TRACE
/* Tracing builds of the library only (make EXTRA=-DQW3_TRACE; the shipped build holds no tracing code): global-timer
 * stamps the pass kernels recorded during the last pass of a stage.  Fused pass: [CTA][layer][16] phase stamps of
 * thread 0 (max_entries = number of values wanted, negative allowed).  Operator-list pass: the time CTA 0 entered each
 * operator plus the end of the pass, or with max_entries < 0 the per-CTA event times [CTA][operator][8]. */
int qw3_debug_trace(qw3_handle h, int32_t stage, uint64_t* out, int32_t max_entries, int32_t* n_entries);
#endif

/* One process per GPU (world > 1, n_stages == world, rank = this process's stage).  Every stage owns
 * a mailbox in its device memory; qw3_stage_export returns its 64-byte CUDA IPC handle, the caller
 * exchanges the handles between the processes (any transport), and qw3_stage_connect maps the mailbox
 * of the next stage (rank+1, wrapping to 0) and of the previous one (rank-1, wrapping).  After that
 * every process calls qw3_generate / qw3_decode_more with the same arguments; hidden states and token
 * ids move between the GPUs by peer stores and device-side flags (replaces copyHiddenBetweenGPUs,
 * Inference.cu:1013-1023).  The generated ids are returned by the last stage's process (n_out = 0
 * elsewhere). */
int qw3_stage_export(qw3_handle h, void* out_handle_64B);
int qw3_stage_connect(qw3_handle h, const void* next_stage_handle_64B, const void* prev_stage_handle_64B);

/* The wait of the stage hand-off protocol (Inference.cu:1013-1023 has no such protocol: it relies on host synchronisation)
 * as a stand-alone launch: one thread waits until *d_flag >= want, at most `limit_clocks` GPU clocks; when the wait runs
 * out the kernel returns and stores `code` in the workspace's error word, which qw3_ws_check reports as QW3_ERR_TIMEOUT.
 * The engine uses the same kernel with a limit of 2^34 clocks; this entry lets a host (or a test) choose a short one. */
int qw3_handoff_wait(const int32_t* d_flag, int32_t want, int64_t limit_clocks, int32_t code, qw3_ws_t ws, void* stream);

/* Row-split tensor parallelism (world > 1, tensor_parallel = 1): one process per GPU; every process loads the whole
 * weight directory, keeps its share of every matrix in the fused pass's layout (its heads of Wqkv / Wo and of the KV
 * cache, its outputs of W1 / inputs of W2, its blocks of the unembedding) and runs ALL layers.  The two reductions per
 * layer cross NVLink inside the pass kernel: partial sums and the gathered hidden state are stored as tagged words into
 * every GPU's exchange buffer (plain peer stores) and polled locally, so each GPU streams 1/world of the weights per
 * token.  The reference has no such mode (its only multi-GPU form is the layer pipeline, Inference.cu:43-47);
 * the pipeline stays available with tensor_parallel = 0.
 * qw3_tp_export returns the 64-byte CUDA IPC handle of this rank's exchange buffer; the caller gathers the handles of
 * all ranks (any transport) and passes them, rank-major (world x 64 bytes), to qw3_tp_connect.  All ranks must have
 * connected before any of them generates, every rank then calls qw3_generate / qw3_decode_more with the same
 * arguments (each returns the ids), and no rank may destroy its handle while another is still generating.  Prompts
 * run token by token through the same kernel, or, with qw3_set_batched_prefill, in blocks that every rank computes in
 * full (the prompt phase is then replicated, not split).  qw3_last_logits returns this rank's blocks of the logits
 * only (NaN elsewhere). */
int qw3_tp_export(qw3_handle h, void* out_handle_64B);
int qw3_tp_connect(qw3_handle h, const void* handles_world_x_64B);

/* Test hooks of the fused token pass (persistent = 2), pure host arithmetic: how it cuts a configuration over `grid`
 * CTAs and `n_ranks` GPUs -- geom_out receives 16 ints {hidden, inter, heads, vocab, n_ranks, rank, heads per rank,
 * CTAs per head, CTAs running the layers, hidden elements owned per CTA, W1 outputs per CTA, vocabulary blocks, grid,
 * 0, 0, 0}, plans_out 5 x 10 ints {CTAs, tiles per CTA, k-steps per CTA, warps along k, tiles per block, blocks per
 * warp, full k-groups, remaining k-steps, bytes per warp stream, ring units per warp} for Wqkv, Wo, W1, W2 and one
 * unembedding block -- and the load-time repack of one matrix (the reference's on-disk layout, Inference.cu:780-900, is
 * unchanged on disk) into the per-(CTA, warp) byte streams the kernel consumes.  QW3_ERR_ARG when the fused pass
 * does not cover the configuration (the engine then keeps the operator-list kernel). */
int qw3_fused_plan(const Qw3Config* cfg, int32_t n_ranks, int32_t rank, int32_t grid, int32_t* geom_out, int32_t* plans_out);
int qw3_fused_repack_host(const Qw3Config* cfg, int32_t n_ranks, int32_t rank, int32_t grid, int32_t op, const void* raw_packed,
                          int64_t out_dim, void* out, int64_t out_bytes);

/* Layers [*first, *first + *count) that stage `stage` of cfg runs (pure host arithmetic). */
int qw3_stage_layers(const Qw3Config* cfg, int32_t stage, int32_t* first, int32_t* count);

#ifdef __cplusplus
}
#endif
#endif
