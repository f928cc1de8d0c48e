// Host engine behind the C handle: the B200 counterpart of class QWen3AWQInfer
// (Inference.cu:356-415).  Same weight directory, same per-layer flow (runOneLayer,
// Inference.cu:1029-1230), same generateResponse contract (Inference.cu:1297-1408), but:
//   * no fp16 copies of the weights (d_dq) and no cuBLAS: five fused kernels per layer;
//   * position, step counter and sampled token live on the device, so a token pass is a fixed
//     launch sequence that is captured once into a CUDA graph and replayed, and the host never
//     waits inside the loops (the reference synchronises six times per token);
//   * the 2-GPU layer split (Inference.cu:43-47) is a list of 1..8 stages; the hidden state and
//     the sampled id move between stages with event-ordered peer copies (the reference's copy is
//     not ordered after the producing stream, Inference.cu:1013-1023).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "fused_pass.h"
#include "pass_flags.h"

namespace qw3 {

int gemv_launch(const W4Desc* d, const Qw3GemvArgs* a, const Workspace* ws, bool pdl, cudaStream_t st);
int attn_decode_launch(const void* q, const void* kc, const void* vc, int heads, int head_dim, long long max_pos,
                       const int* d_pos, int pos, void* ctx, const Workspace* ws, bool pdl, cudaStream_t st);
int embed_gather_launch(const void* packed, const void* scale, const void* zp, long long n_alloc, long long hidden,
                        long long vocab, const int* d_token, const int* d_index, const int* d_skip, int token, void* out,
                        bool pdl, cudaStream_t st);
int embed_rows_launch(const void* packed, const void* scale, const void* zp, long long n_alloc, int hidden, long long vocab,
                      const int* d_tokens, int rows, void* out, cudaStream_t st);
int rmsnorm_rows_launch(const void* x, const void* gamma, int n, float eps, int rows, void* out, cudaStream_t st);
int rope_kv_rows_launch(void* qkv, void* kc, void* vc, const void* cos_t, const void* sin_t, int hidden, long long max_pos,
                        int pos0, int rows, cudaStream_t st);
int attn_prefill_launch(const void* qkv, const void* kc, const void* vc, int heads, int hidden, long long max_pos, int pos0,
                        int rows, void* ctx, cudaStream_t st);
int gemm_launch(qw3_w4_t w, const void* d_x, int64_t rows, void* d_y, qw3_ws_t ws, void* stream, int epilogue);
int step_tail_launch(int* d_pos, int* d_step, const int* d_token, int* d_out_ids, int* d_skip, int* d_epoch, bool pdl,
                     cudaStream_t st);
const W4Desc* w4_desc(qw3_w4_t w);
const Workspace* ws_struct(qw3_ws_t ws);
int flag_wait_launch(const int* d_flag, int want, long long limit_clocks, int* err, int code, cudaStream_t st);
// stage hand-off between processes (handoff.cu)
size_t mailbox_bytes(int hidden);
void* mailbox_linked_inbox(void* mb, int hidden);
void* mailbox_token_word(void* mb);
int block_send(const void* rows_src, size_t bytes, void* next_mb, const void* my_mb, int msg, int hidden, int* err, cudaStream_t st);
int block_recv(void* rows_dst, size_t bytes, void* my_mb, void* prev_mb, int msg, int hidden, int* err, cudaStream_t st);
int handoff_send(const void* hidden, void* next_mb, const void* my_mb, int msg, int hidden_n, int* err, cudaStream_t st);
int handoff_recv(void* hidden, const void* my_mb, void* prev_mb, int msg, int hidden_n, int* err, cudaStream_t st);
int token_send(const int* d_token, void* first_mb, int msg, cudaStream_t st);
int token_recv(int* d_token, const void* my_mb, int msg, int* err, cudaStream_t st);
// persistent token-pass kernel (decode_pass.cu)
struct PassOp;
int pass_init_device();
bool pass_supports(const W4Desc* d);
size_t pass_op_bytes();
void pass_fill_gemv(PassOp* op, const W4Desc* d, const void* x, const void* gamma, float eps, int epilogue, void* y,
                    void* kc, void* vc);
void pass_fill_attn(PassOp* op, const void* q, void* kc, void* vc, void* ctx, int heads);
void pass_fill_embed(PassOp* op, const void* packed, const void* scale, const void* zp, long long n_alloc, void* hidden_out,
                     int hidden);
size_t pass_xchg_bytes();
void pass_link(PassOp* op, int flags, int src, const void* xt, void* yt, const void* rt, int rsrc);
int pass_launch(const void* d_ops, int n_ops, int* d_done, unsigned long long* d_xchg, const int* d_epoch, const int* d_pos, const int* d_token, const int* d_skip,
                const int* d_prompt, int decode, const void* cos_t, const void* sin_t, int heads, int hidden,
                long long max_pos, long long vocab, int* d_token_out, float* logits_f32, unsigned long long* trace,
                unsigned long long* trace2, const int* d_gen, const void* tok_in, const void* tok_out_slot, const Workspace* ws, cudaStream_t st);

#define QW3_TRY(expr)                     \
    do {                                  \
        int rc__ = (expr);                \
        if (rc__ != QW3_OK) return rc__;  \
    } while (0)

struct W4Dev {  // AWQWeight (Inference.cu:318-325) minus d_dq
    void* packed = nullptr;
    void* scale = nullptr;
    void* zp = nullptr;
    qw3_w4_t desc = nullptr;
    int64_t out_dim = 0, in_dim = 0, n_alloc = 0;
};

struct LayerDev {
    W4Dev wqkv, wo, w1, w2;
    void* gamma = nullptr;
    void* kc = nullptr;
    void* vc = nullptr;
};

struct Stage {  // GPUContext (Inference.cu:328-351) for one pipeline stage
    int device = 0;
    int gidx = 0;                      // index of this stage in the whole pipeline
    int l0 = 0, l1 = 0;
    cudaStream_t stream = nullptr;
    qw3_ws_t ws = nullptr;
    std::vector<LayerDev> layers;
    void *hidden = nullptr, *q = nullptr, *ctx = nullptr, *mlp = nullptr;
    void *cos_t = nullptr, *sin_t = nullptr;
    int *d_pos = nullptr, *d_step = nullptr, *d_token = nullptr, *d_skip = nullptr;
    int *d_prompt = nullptr, *d_out_ids = nullptr;
    W4Dev emb, unemb;                  // first / last stage only
    void* logits16 = nullptr;          // last stage
    float* logits32 = nullptr;         // last stage, keep_logits
    cudaEvent_t done = nullptr;        // recorded after each token pass of this stage
    cudaEvent_t taken = nullptr;       // recorded after this stage has copied its input from a peer
    cudaGraphExec_t g_prompt = nullptr, g_decode = nullptr;
    int launches_prompt = 0, launches_decode = 0;
    // persistent pass: operator lists (device) of the prompt pass and of the decode pass
    void* ops_prompt = nullptr;
    void* ops_decode = nullptr;
    int n_ops_prompt = 0, n_ops_decode = 0;
    // one process per GPU: decode pass whose first / last operators poll / store the neighbours' mailboxes themselves
    void* ops_linked = nullptr;
    int n_ops_linked = 0;
    cudaGraphExec_t g_linked = nullptr;
    int launches_linked = 0;
    int* d_gen = nullptr;                        // generation counter of the sequence (part of the cross-GPU tags)
    unsigned long long** d_tok_out_slot = nullptr;   // last stage: holds the address of the first stage's token word
    int* d_done = nullptr;    // persistent pass: per-operator arrival counters + the launch epoch word behind them
    int* d_epoch = nullptr;
    unsigned long long* d_xchg = nullptr;   // tagged partial sums exchanged between CTAs
    unsigned long long *hidden_t = nullptr, *ctx_t = nullptr, *mlp_t = nullptr, *qkv_t = nullptr;   // tagged activations, one word per pair
    unsigned long long* d_trace = nullptr;   // per-operator entry times of the last pass (debug)
    unsigned long long* d_trace2 = nullptr;  // per-CTA event times of the last pass (debug)
    bool persistent = false;
    FusedPass* fused = nullptr;   // fused token pass (persistent = 2): paired operators, repacked weight streams
    // batched prompt phase: activations of a block of PF_BLOCK prompt rows (allocated at the first use)
    void *pf_h = nullptr, *pf_n = nullptr, *pf_qkv = nullptr, *pf_ctx = nullptr, *pf_mlp = nullptr;
};

}  // namespace qw3

using namespace qw3;

struct qw3_engine {
    Qw3Config cfg;
    std::vector<Stage> st;
    std::vector<void*> allocs;          // every cudaMalloc, with its device
    std::vector<int> alloc_dev;
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr;  // on stage 0's device
    float prompt_ms = 0.f, decode_ms = 0.f;
    int64_t launches = 0;
    // one process per GPU: this stage's mailbox and the ring neighbours' (mapped through CUDA IPC)
    void* mailbox = nullptr;
    void* next_mb = nullptr;
    void* prev_mb = nullptr;
    bool next_is_prev = false;
    int msg_out = 0, msg_in = 0;        // hidden-state messages sent to the next stage / taken from the previous one
    int tok_out = 0, tok_in = 0;        // token messages (last stage -> first stage)
    int blk_out = 0, blk_in = 0;        // blocks of prompt rows (batched prompt phase)
    int batched_prefill = -1;           // prompt in blocks of rows through the tensor-core contraction: 1 always, 0 never (the reference's
                                        // token loop), -1 (default) from PF_AUTO_ROWS prompt tokens on (qw3_set_batched_prefill)
    int seq_len = 0;                    // token passes through the layers so far (next position)
    int sampled = 0;                    // ids sampled since the last prompt
    int gen = 0;                        // generate calls so far (one process per GPU: part of the cross-GPU tags)
    bool linked_now = false;            // the pass being enqueued is a chained decode pass (ops_linked)
    bool chain_decode = true;           // qw3_set_chained_decode
    std::vector<void*> tp_peers;        // row-split over GPUs: the other ranks' exchange buffers (CUDA IPC mappings)
    bool tp_connected = false;
};

namespace qw3 {

static int dev_alloc(qw3_engine* e, int dev, void** p, size_t bytes) {
    QW3_CUDA(cudaSetDevice(dev));
    cudaError_t r = cudaMalloc(p, bytes);
    if (r != cudaSuccess) {
        set_last_error("cudaMalloc(%zu bytes) on device %d -> %s", bytes, dev, cudaGetErrorString(r));
        return r == cudaErrorMemoryAllocation ? QW3_ERR_NOMEM : QW3_ERR_CUDA;
    }
    e->allocs.push_back(*p);
    e->alloc_dev.push_back(dev);
    return QW3_OK;
}

// readBinaryFileToDevice (Inference.cu:297-311): the file must hold at least `bytes`; excess is ignored.
static int read_to_device(qw3_engine* e, const std::string& fn, void* d_ptr, size_t bytes, cudaStream_t st,
                          std::vector<uint16_t>* keep_host = nullptr) {
    FILE* f = std::fopen(fn.c_str(), "rb");
    if (!f) {
        set_last_error("could not open %s", fn.c_str());
        return QW3_ERR_IO;
    }
    if (bytes > e->pinned_bytes) {
        if (e->pinned) cudaFreeHost(e->pinned);
        e->pinned = nullptr;
        e->pinned_bytes = 0;
        QW3_CUDA(cudaMallocHost(&e->pinned, bytes));
        e->pinned_bytes = bytes;
    }
    const size_t got = std::fread(e->pinned, 1, bytes, f);
    std::fclose(f);
    if (got != bytes) {
        set_last_error("read failed for %s: wanted %zu bytes, got %zu", fn.c_str(), bytes, got);
        return QW3_ERR_IO;
    }
    if (keep_host) {
        keep_host->resize(bytes / 2);
        std::memcpy(keep_host->data(), e->pinned, bytes);
    }
    QW3_CUDA(cudaMemcpyAsync(d_ptr, e->pinned, bytes, cudaMemcpyHostToDevice, st));
    QW3_CUDA(cudaStreamSynchronize(st));  // the staging buffer is reused by the next file
    return QW3_OK;
}

static float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1u, ex = (h >> 10) & 31u, man = h & 1023u;
    float v;
    if (ex == 0) v = std::ldexp((float)man, -24);
    else if (ex == 31) v = man ? NAN : INFINITY;
    else v = std::ldexp((float)(man | 1024u), (int)ex - 25);
    return sign ? -v : v;
}

// Every zero-point an integer of magnitude <= 1023: 1024 + zp and 64 + zp are then exact in fp16.
static int zp_all_integral(const std::vector<uint16_t>& zp) {
    for (uint16_t h : zp) {
        const float v = half_bits_to_float(h);
        if (!(std::fabs(v) <= 1023.0f) || v != std::floor(v)) return 0;
    }
    return 1;
}

// One AWQ matrix: allocation sizes as Inference.cu:616-626, file names as Inference.cu:780-900.
static int load_w4(qw3_engine* e, Stage& s, W4Dev& w, int64_t out_dim, int64_t in_dim, const std::string& fp,
                   const std::string& fs, const std::string& fz, bool make_desc) {
    w.out_dim = out_dim; w.in_dim = in_dim; w.n_alloc = out_dim / 128;
    const size_t pbytes = (size_t)out_dim * ((in_dim + 1) / 2), gbytes = (size_t)w.n_alloc * 2;
    QW3_TRY(dev_alloc(e, s.device, &w.packed, pbytes));
    QW3_TRY(dev_alloc(e, s.device, &w.scale, gbytes));
    QW3_TRY(dev_alloc(e, s.device, &w.zp, gbytes));
    std::vector<uint16_t> zp_host;
    QW3_TRY(read_to_device(e, fp, w.packed, pbytes, s.stream));
    QW3_TRY(read_to_device(e, fs, w.scale, gbytes, s.stream));
    QW3_TRY(read_to_device(e, fz, w.zp, gbytes, s.stream, &zp_host));
    if (make_desc)
        QW3_TRY(qw3_w4_create(w.packed, w.scale, w.zp, w.n_alloc, out_dim, in_dim, zp_all_integral(zp_host), &w.desc));
    return QW3_OK;
}

static int validate_config(Qw3Config& c) {
    QW3_REQUIRE(c.head_dim == 128, "config: head_dim must be 128");
    QW3_REQUIRE(c.hidden == c.heads * c.head_dim, "config: hidden must equal heads*head_dim");
    QW3_REQUIRE(c.hidden % 128 == 0 && c.inter % 128 == 0 && c.vocab % 128 == 0, "config: hidden, inter and vocab must be multiples of 128");
    QW3_REQUIRE(c.layers >= 1 && c.max_pos >= 2, "config: layers >= 1 and max_pos >= 2 required");
    QW3_REQUIRE(c.n_stages >= 1 && c.n_stages <= QW3_MAX_STAGES && c.n_stages <= c.layers, "config: n_stages must be in 1..min(8, layers)");
    QW3_REQUIRE(c.world >= 1 && c.rank >= 0 && c.rank < c.world, "config: bad rank/world");
    bool any = false;
    for (int s = 0; s <= c.n_stages; ++s) any |= c.first_layer[s] != 0;
    if (!any) {  // even split, remainder on the leading stages: 36 layers on 8 stages -> 5,5,5,5,4,4,4,4
        const int base = c.layers / c.n_stages, rem = c.layers % c.n_stages;
        int l = 0;
        for (int s = 0; s < c.n_stages; ++s) {
            c.first_layer[s] = l;
            l += base + (s < rem ? 1 : 0);
        }
        c.first_layer[c.n_stages] = c.layers;
    }
    QW3_REQUIRE(c.first_layer[0] == 0 && c.first_layer[c.n_stages] == c.layers, "config: stage split must cover all layers");
    for (int s = 0; s < c.n_stages; ++s)
        QW3_REQUIRE(c.first_layer[s] < c.first_layer[s + 1], "config: every stage needs at least one layer");
    return QW3_OK;
}

// One decoder layer for one token, five launches (runOneLayer, Inference.cu:1029-1230).
static int enqueue_layer(qw3_engine* e, Stage& s, int li, bool pdl, int* launches) {
    const Qw3Config& c = e->cfg;
    LayerDev& L = s.layers[li];
    const Workspace* ws = ws_struct(s.ws);
    Qw3GemvArgs a;
    // RMSNorm + Wqkv + split + RoPE + KV append (Inference.cu:1036-1103)
    std::memset(&a, 0, sizeof(a));
    a.d_x = s.hidden; a.d_gamma = L.gamma; a.eps = c.eps; a.epilogue = QW3_EPI_ROPE_KV; a.d_y = s.q;
    a.d_k_cache = L.kc; a.d_v_cache = L.vc; a.d_cos = s.cos_t; a.d_sin = s.sin_t;
    a.heads = c.heads; a.head_dim = c.head_dim; a.max_pos = c.max_pos; a.d_pos = s.d_pos;
    QW3_TRY(gemv_launch(w4_desc(L.wqkv.desc), &a, ws, pdl, s.stream));
    // attention over rows 0..pos (Inference.cu:1106-1120, length repaired to pos+1 in every layer)
    QW3_TRY(attn_decode_launch(s.q, L.kc, L.vc, c.heads, c.head_dim, c.max_pos, s.d_pos, 0, s.ctx, ws, pdl, s.stream));
    // Wo + residual (Inference.cu:1122-1156; reads ctx, never in place)
    std::memset(&a, 0, sizeof(a));
    a.d_x = s.ctx; a.epilogue = QW3_EPI_RESIDUAL; a.d_y = s.hidden;
    QW3_TRY(gemv_launch(w4_desc(L.wo.desc), &a, ws, pdl, s.stream));
    // RMSNorm (same gamma) + W1 + GeLU (Inference.cu:1158-1197)
    std::memset(&a, 0, sizeof(a));
    a.d_x = s.hidden; a.d_gamma = L.gamma; a.eps = c.eps; a.epilogue = QW3_EPI_GELU; a.d_y = s.mlp;
    QW3_TRY(gemv_launch(w4_desc(L.w1.desc), &a, ws, pdl, s.stream));
    // W2 + residual (Inference.cu:1198-1228)
    std::memset(&a, 0, sizeof(a));
    a.d_x = s.mlp; a.epilogue = QW3_EPI_RESIDUAL; a.d_y = s.hidden;
    QW3_TRY(gemv_launch(w4_desc(L.w2.desc), &a, ws, pdl, s.stream));
    *launches += 5;
    return QW3_OK;
}

// Final norm with the last layer's gamma + unembed + arg-max (sampleNextToken, Inference.cu:1235-1292).
static int enqueue_sample(qw3_engine* e, Stage& s, bool pdl, int* launches) {
    const Qw3Config& c = e->cfg;
    Qw3GemvArgs a;
    std::memset(&a, 0, sizeof(a));
    a.d_x = s.hidden; a.d_gamma = s.layers.back().gamma; a.eps = c.eps; a.epilogue = QW3_EPI_ARGMAX;
    a.d_y = s.logits16; a.d_token = s.d_token; a.d_logits_f32 = s.logits32;
    QW3_TRY(gemv_launch(w4_desc(s.unemb.desc), &a, ws_struct(s.ws), pdl, s.stream));
    *launches += 1;
    return QW3_OK;
}

// The launch sequence of one token pass on one stage.
static int enqueue_stage_pass(qw3_engine* e, int si, bool decode, bool layers, bool pdl, int* launches) {
    const Qw3Config& c = e->cfg;
    Stage& s = e->st[si];
    const bool first = e->st[si].gidx == 0, last = e->st[si].gidx == c.n_stages - 1;
    QW3_CUDA(cudaSetDevice(s.device));
    if (layers && s.fused) {
        // the whole pass of this stage is one cooperative launch of the fused kernel
        QW3_TRY(fused_launch(s.fused, decode ? 1 : 0, s.stream));
        *launches += 1;
    } else if (layers && s.persistent) {
        // the whole pass of this stage is one cooperative launch
        const bool linked = decode && e->linked_now;
        const void* ops = linked ? s.ops_linked : (decode ? s.ops_decode : s.ops_prompt);
        const int n_ops = linked ? s.n_ops_linked : (decode ? s.n_ops_decode : s.n_ops_prompt);
        QW3_TRY(pass_launch(ops, n_ops, s.d_done, s.d_xchg, s.d_epoch, s.d_pos, s.d_token, first ? s.d_skip : nullptr, s.d_prompt,
                            decode ? 1 : 0, s.cos_t, s.sin_t, c.heads, c.hidden, c.max_pos, c.vocab, s.d_token, s.logits32, s.d_trace,
                            s.d_trace2, s.d_gen, (e->mailbox && first) ? mailbox_token_word(e->mailbox) : nullptr,
                            (decode && last) ? s.d_tok_out_slot : nullptr, ws_struct(s.ws), s.stream));
        *launches += 1;
    } else if (layers) {
        if (first) {
            if (decode)
                QW3_TRY(embed_gather_launch(s.emb.packed, s.emb.scale, s.emb.zp, s.emb.n_alloc, c.hidden, c.vocab, s.d_token,
                                            nullptr, s.d_skip, 0, s.hidden, pdl, s.stream));
            else
                QW3_TRY(embed_gather_launch(s.emb.packed, s.emb.scale, s.emb.zp, s.emb.n_alloc, c.hidden, c.vocab, s.d_prompt,
                                            s.d_pos, nullptr, 0, s.hidden, pdl, s.stream));
            *launches += 1;
        }
        for (int li = 0; li < (int)s.layers.size(); ++li) QW3_TRY(enqueue_layer(e, s, li, pdl, launches));
    }
    if (decode && last && !(layers && (s.persistent || s.fused))) QW3_TRY(enqueue_sample(e, s, pdl, launches));
    QW3_TRY(step_tail_launch(layers ? s.d_pos : nullptr, (decode && last) ? s.d_step : nullptr, s.d_token,
                             (decode && last) ? s.d_out_ids : nullptr, first ? s.d_skip : nullptr,
                             (layers && s.persistent && !s.fused) ? s.d_epoch : nullptr, pdl, s.stream));
    *launches += 1;
    return QW3_OK;
}

// Operator list of one pass of a stage, uploaded once (runOneLayer's sequence, Inference.cu:1029-1230).
// `linked` (one process per GPU, decode): the first operators read the hidden state from this stage's tagged inbox,
// which the stage before stores from its GPU, the last residual operator stores its tagged output into the next
// stage's inbox, and the embedding takes the sampled id from the tagged token word.
static int build_pass_program(qw3_engine* e, int si, bool decode, void** d_ops, int* n_ops, bool linked = false) {
    const Qw3Config& c = e->cfg;
    Stage& s = e->st[si];
    const bool first = e->st[si].gidx == 0, last = e->st[si].gidx == c.n_stages - 1;
    const size_t ob = pass_op_bytes();
    const int n = (first ? 1 : 0) + 5 * (int)s.layers.size() + ((decode && last) ? 1 : 0);
    std::vector<uint8_t> host((size_t)n * ob + 256);
    uint8_t* base = host.data();
    base += (256 - (reinterpret_cast<uintptr_t>(base) & 255)) & 255;   // descriptors hold 64-byte aligned tensor maps
    int k = 0;
    auto at = [&](int i) { return reinterpret_cast<PassOp*>(base + (size_t)i * ob); };
    // Inside a launch activations go from operator to operator as tagged words (hidden_t, qkv_t, ctx_t, mlp_t); only
    // the final arg-max waits on an arrival counter (the unembedding's).
    constexpr int PUBLISH = PASS_PUBLISH, PEER_OUT = PASS_PEER_OUT, TOKEN_PEER = PASS_TOKEN_PEER, SRC_PEER = P_SRC_PEER;
    bool hidden_tagged = false;            // hidden_t holds the residual stream (written in this launch)
    int hidden_src = -1;                   // operator that wrote it last
    const unsigned long long* hidden_in = s.hidden_t;   // where the tagged residual stream is read from
    if (linked && !first) {
        hidden_in = static_cast<const unsigned long long*>(mailbox_linked_inbox(e->mailbox, c.hidden));
        hidden_tagged = true;
        hidden_src = SRC_PEER;
    }
    void* const peer_inbox = (linked && !last) ? mailbox_linked_inbox(e->next_mb, c.hidden) : nullptr;
    const int n_layers = (int)s.layers.size();
    int li = 0;
    if (first) {
        pass_fill_embed(at(k), s.emb.packed, s.emb.scale, s.emb.zp, s.emb.n_alloc, s.hidden, c.hidden);
        pass_link(at(k), linked ? TOKEN_PEER : 0, -1, nullptr, s.hidden_t, nullptr, -1);
        hidden_src = k;
        ++k;
        hidden_tagged = true;
    }
    for (LayerDev& L : s.layers) {
        pass_fill_gemv(at(k), w4_desc(L.wqkv.desc), s.hidden, L.gamma, c.eps, QW3_EPI_ROPE_KV, s.q, L.kc, L.vc);
        pass_link(at(k), 0, hidden_src == SRC_PEER ? SRC_PEER : k - 1, hidden_tagged ? hidden_in : nullptr, s.qkv_t, nullptr, -1);
        ++k;
        pass_fill_attn(at(k), s.q, L.kc, L.vc, s.ctx, c.heads);
        pass_link(at(k), 0, k - 1, s.qkv_t, s.ctx_t, nullptr, -1);
        ++k;
        pass_fill_gemv(at(k), w4_desc(L.wo.desc), s.ctx, nullptr, c.eps, QW3_EPI_RESIDUAL, s.hidden, nullptr, nullptr);
        pass_link(at(k), 0, k - 1, s.ctx_t, s.hidden_t, hidden_tagged ? hidden_in : nullptr, hidden_src);
        hidden_src = k;
        hidden_in = s.hidden_t;
        ++k;
        hidden_tagged = true;
        pass_fill_gemv(at(k), w4_desc(L.w1.desc), s.hidden, L.gamma, c.eps, QW3_EPI_GELU, s.mlp, nullptr, nullptr);
        pass_link(at(k), 0, k - 1, s.hidden_t, s.mlp_t, nullptr, -1);
        ++k;
        pass_fill_gemv(at(k), w4_desc(L.w2.desc), s.mlp, nullptr, c.eps, QW3_EPI_RESIDUAL, s.hidden, nullptr, nullptr);
        if (peer_inbox != nullptr && li == n_layers - 1)   // the stage's result goes straight into the next stage's inbox
            pass_link(at(k), PEER_OUT, k - 1, s.mlp_t, peer_inbox, s.hidden_t, hidden_src);
        else
            pass_link(at(k), 0, k - 1, s.mlp_t, s.hidden_t, s.hidden_t, hidden_src);
        hidden_src = k;
        ++k;
        ++li;
    }
    if (decode && last) {
        pass_fill_gemv(at(k), w4_desc(s.unemb.desc), s.hidden, s.layers.back().gamma, c.eps, QW3_EPI_ARGMAX, s.logits16,
                       nullptr, nullptr);
        pass_link(at(k), PUBLISH, k - 1, hidden_tagged ? s.hidden_t : nullptr, nullptr, nullptr, -1);
        ++k;
    }
    QW3_TRY(dev_alloc(e, s.device, d_ops, (size_t)n * ob));
    QW3_CUDA(cudaMemcpy(*d_ops, base, (size_t)n * ob, cudaMemcpyHostToDevice));
    *n_ops = n;
    return QW3_OK;
}

static int capture_stage_graph(qw3_engine* e, int si, bool decode, cudaGraphExec_t* out, int* launches) {
    Stage& s = e->st[si];
    QW3_CUDA(cudaSetDevice(s.device));
    QW3_CUDA(cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeThreadLocal));
    *launches = 0;
    int rc = enqueue_stage_pass(e, si, decode, true, e->cfg.use_pdl != 0, launches);   // e->linked_now selects the chained program
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(s.stream, &g);
    if (rc != QW3_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    QW3_CUDA(ce);
    ce = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    QW3_CUDA(ce);
    return QW3_OK;
}

// Hidden state (and, towards stage 0, the sampled id) from stage `from` to stage `to`, ordered
// after the producer's pass by an event (copyHiddenBetweenGPUs, Inference.cu:1013-1023).
static int handoff(qw3_engine* e, int from, int to, bool hidden, bool token) {
    Stage &a = e->st[from], &b = e->st[to];
    QW3_CUDA(cudaSetDevice(b.device));
    QW3_CUDA(cudaStreamWaitEvent(b.stream, a.done, 0));
    if (hidden)
        QW3_CUDA(cudaMemcpyPeerAsync(b.hidden, b.device, a.hidden, a.device, (size_t)e->cfg.hidden * 2, b.stream));
    if (token) QW3_CUDA(cudaMemcpyPeerAsync(b.d_token, b.device, a.d_token, a.device, 4, b.stream));
    // The producer may not overwrite what is being copied: its next pass waits for the copy.
    QW3_CUDA(cudaEventRecord(b.taken, b.stream));
    QW3_CUDA(cudaSetDevice(a.device));
    QW3_CUDA(cudaStreamWaitEvent(a.stream, b.taken, 0));
    return QW3_OK;
}

constexpr int PF_AUTO_ROWS = 16;   // prompts at least this long take the batched prompt phase unless the caller chose
static bool use_batched_prefill(const qw3_engine* e, int n_prompt) {
    return e->batched_prefill > 0 || (e->batched_prefill < 0 && n_prompt >= PF_AUTO_ROWS);
}

// ---- batched prompt phase ---------------------------------------------------------------------------
// A block of `rows` prompt tokens at positions pos0.. goes through every stage together: the projections are
// the tensor-core contraction, the rest the row kernels of prefill.cu.  Same per-element arithmetic as the
// token-at-a-time loop (Inference.cu:1304-1343); the contractions sum in a different fp32 order.
constexpr int PF_BLOCK = 2048;  // also the rows a block inbox of the mailbox holds (handoff.cu); the contraction reaches 0.4 of its
                                // tensor bound at 256 rows and 0.6 at 2048

static int prefill_alloc(qw3_engine* e, Stage& s) {
    if (s.pf_h) return QW3_OK;
    const Qw3Config& c = e->cfg;
    const size_t H = (size_t)c.hidden * 2 * PF_BLOCK, I = (size_t)c.inter * 2 * PF_BLOCK;
    QW3_TRY(dev_alloc(e, s.device, &s.pf_h, H));
    QW3_TRY(dev_alloc(e, s.device, &s.pf_n, H));
    QW3_TRY(dev_alloc(e, s.device, &s.pf_qkv, 3 * H));
    QW3_TRY(dev_alloc(e, s.device, &s.pf_ctx, H));
    QW3_TRY(dev_alloc(e, s.device, &s.pf_mlp, I));
    return QW3_OK;
}

// One stage's share of a block: its layers over `rows` rows in s.pf_h (the first stage gathers the embeddings first),
// then what the token loop leaves behind: the last row's hidden state and the position counter.
static int prefill_stage_block(qw3_engine* e, Stage& s, int t0, int rows) {
    const Qw3Config& c = e->cfg;
    const int H = c.hidden;
    if (s.gidx == 0) {
        QW3_TRY(embed_rows_launch(s.emb.packed, s.emb.scale, s.emb.zp, s.emb.n_alloc, H, c.vocab, s.d_prompt + t0, rows, s.pf_h,
                                  s.stream));
        e->launches += 1;
    }
    for (LayerDev& L : s.layers) {
        QW3_TRY(rmsnorm_rows_launch(s.pf_h, L.gamma, H, c.eps, rows, s.pf_n, s.stream));
        QW3_TRY(qw3_gemm_w4a16(L.wqkv.desc, s.pf_n, rows, s.pf_qkv, s.ws, s.stream));
        QW3_TRY(rope_kv_rows_launch(s.pf_qkv, L.kc, L.vc, s.cos_t, s.sin_t, H, c.max_pos, t0, rows, s.stream));
        QW3_TRY(attn_prefill_launch(s.pf_qkv, L.kc, L.vc, c.heads, H, c.max_pos, t0, rows, s.pf_ctx, s.stream));
        QW3_TRY(gemm_launch(L.wo.desc, s.pf_ctx, rows, s.pf_h, s.ws, s.stream, QW3_EPI_RESIDUAL));
        QW3_TRY(rmsnorm_rows_launch(s.pf_h, L.gamma, H, c.eps, rows, s.pf_n, s.stream));
        QW3_TRY(gemm_launch(L.w1.desc, s.pf_n, rows, s.pf_mlp, s.ws, s.stream, QW3_EPI_GELU));
        QW3_TRY(gemm_launch(L.w2.desc, s.pf_mlp, rows, s.pf_h, s.ws, s.stream, QW3_EPI_RESIDUAL));
        e->launches += 7;
    }
    QW3_CUDA(cudaMemcpyAsync(s.hidden, static_cast<char*>(s.pf_h) + (size_t)(rows - 1) * H * 2, (size_t)H * 2,
                             cudaMemcpyDeviceToDevice, s.stream));
    const int next_pos[4] = {t0 + rows, 0, 0, 0};
    QW3_CUDA(cudaMemcpyAsync(s.d_pos, next_pos, 4, cudaMemcpyHostToDevice, s.stream));
    return QW3_OK;
}

// Single process: the block goes through the stages one after another.
static int prefill_block(qw3_engine* e, int t0, int rows) {
    const Qw3Config& c = e->cfg;
    const int N = c.n_stages, H = c.hidden;
    for (int si = 0; si < N; ++si) {
        Stage& s = e->st[si];
        QW3_TRY(prefill_alloc(e, s));
        QW3_CUDA(cudaSetDevice(s.device));
        if (si > 0) {   // the block's hidden rows from the stage before, ordered by events as the one-row hand-off
            Stage& a = e->st[si - 1];
            QW3_CUDA(cudaStreamWaitEvent(s.stream, a.done, 0));
            QW3_CUDA(cudaMemcpyPeerAsync(s.pf_h, s.device, a.pf_h, a.device, (size_t)rows * H * 2, s.stream));
            QW3_CUDA(cudaEventRecord(s.taken, s.stream));
            QW3_CUDA(cudaSetDevice(a.device));
            QW3_CUDA(cudaStreamWaitEvent(a.stream, s.taken, 0));
            QW3_CUDA(cudaSetDevice(s.device));
        }
        QW3_TRY(prefill_stage_block(e, s, t0, rows));
        QW3_CUDA(cudaEventRecord(s.done, s.stream));
    }
    return QW3_OK;
}

// One process per GPU: this stage takes the block from the stage before through its block inbox (the stages overlap
// on successive blocks: two inbox slots, acknowledged), runs its layers and hands the rows on.
static int prefill_block_mp(qw3_engine* e, int t0, int rows) {
    const Qw3Config& c = e->cfg;
    Stage& s = e->st[0];
    const bool first = s.gidx == 0, last = s.gidx == c.n_stages - 1;
    const size_t bytes = (size_t)rows * c.hidden * 2;
    QW3_TRY(prefill_alloc(e, s));
    QW3_CUDA(cudaSetDevice(s.device));
    if (!first) {
        QW3_TRY(block_recv(s.pf_h, bytes, e->mailbox, e->prev_mb, ++e->blk_in, c.hidden, ws_struct(s.ws)->err, s.stream));
        e->launches += 2;
    }
    QW3_TRY(prefill_stage_block(e, s, t0, rows));
    if (!last) {
        QW3_TRY(block_send(s.pf_h, bytes, e->next_mb, e->mailbox, ++e->blk_out, c.hidden, ws_struct(s.ws)->err, s.stream));
        e->launches += 2;
    }
    return QW3_OK;
}

static int run_pass(qw3_engine* e, bool decode, bool layers) {
    const Qw3Config& c = e->cfg;
    const int N = c.n_stages;
    for (int si = 0; si < N; ++si) {
        Stage& s = e->st[si];
        if (si > 0 && layers) QW3_TRY(handoff(e, si - 1, si, true, false));
        if (!layers && si != N - 1) continue;  // sample-only pass touches the last stage alone
        QW3_CUDA(cudaSetDevice(s.device));
        cudaGraphExec_t g = decode ? s.g_decode : s.g_prompt;
        if (layers && g) {
            QW3_CUDA(cudaGraphLaunch(g, s.stream));
            e->launches += decode ? s.launches_decode : s.launches_prompt;
        } else {
            int n = 0;
            QW3_TRY(enqueue_stage_pass(e, si, decode, layers, false, &n));
            e->launches += n;
        }
        QW3_CUDA(cudaEventRecord(s.done, s.stream));
    }
    return QW3_OK;
}

}  // namespace qw3

extern "C" {

int qw3_config_default(Qw3Config* c) {
    QW3_REQUIRE(c, "qw3_config_default: null pointer");
    std::memset(c, 0, sizeof(*c));
    c->hidden = 4096; c->inter = 12288; c->heads = 32; c->head_dim = 128; c->layers = 36; c->vocab = 151936;
    c->max_pos = 40960; c->eps = 1e-6f; c->rope_base = 10000.0f; c->sample_first = 0;
    c->n_stages = 1; c->rank = 0; c->world = 1; c->use_graph = 1; c->use_pdl = 1; c->keep_logits = 0; c->persistent = 2;
    c->attn_split_min = 0;
    return QW3_OK;
}

int qw3_destroy(qw3_handle e) {
    if (!e) return QW3_OK;
    for (Stage& s : e->st) {
        cudaSetDevice(s.device);
        if (s.stream) cudaStreamSynchronize(s.stream);
        if (s.g_prompt) cudaGraphExecDestroy(s.g_prompt);
        if (s.g_decode) cudaGraphExecDestroy(s.g_decode);
        if (s.g_linked) cudaGraphExecDestroy(s.g_linked);
        if (s.fused) fused_destroy(s.fused);
        for (LayerDev& L : s.layers) {
            qw3_w4_destroy(L.wqkv.desc); qw3_w4_destroy(L.wo.desc); qw3_w4_destroy(L.w1.desc); qw3_w4_destroy(L.w2.desc);
        }
        qw3_w4_destroy(s.unemb.desc);
        if (s.ws) qw3_ws_destroy(s.ws);
        if (s.done) cudaEventDestroy(s.done);
        if (s.taken) cudaEventDestroy(s.taken);
        if (s.stream) cudaStreamDestroy(s.stream);
    }
    if (!e->st.empty()) cudaSetDevice(e->st[0].device);
    for (void* pm : e->tp_peers)
        if (pm) cudaIpcCloseMemHandle(pm);
    if (e->next_mb) cudaIpcCloseMemHandle(e->next_mb);
    if (e->prev_mb && !e->next_is_prev) cudaIpcCloseMemHandle(e->prev_mb);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->ev2) cudaEventDestroy(e->ev2);
    for (size_t i = 0; i < e->allocs.size(); ++i) {
        cudaSetDevice(e->alloc_dev[i]);
        cudaFree(e->allocs[i]);
    }
    if (e->pinned) cudaFreeHost(e->pinned);
    delete e;
    return QW3_OK;
}

// The fused token pass of one stage, when its shapes are covered (else the stage keeps the operator-list kernel).
static int create_fused(qw3_engine* e, Stage& s) {
    const Qw3Config& c = e->cfg;
    const Workspace* ws = ws_struct(s.ws);
    const int n_layers = (int)s.layers.size();
    FusedGeom g;
    FGemvPlan plans[F_NOPS];
    const bool tp = c.tensor_parallel != 0 && c.world > 1;
    const int n_ranks = tp ? c.world : 1, rank = tp ? c.rank : 0;
    if (!fused_plan(c.hidden, c.inter, c.heads, c.vocab, n_layers, c.max_pos, n_ranks, rank, ws->sm_count, &g, plans)) {
        if (tp) {
            set_last_error("tensor_parallel: the fused pass does not cover this configuration on %d GPUs", n_ranks);
            return QW3_ERR_ARG;
        }
        return QW3_OK;
    }
    auto mat = [](const W4Dev& w) {
        FusedMatrix m;
        m.packed = w.packed; m.scale = w.scale; m.zp = w.zp; m.n_alloc = w.n_alloc; m.out_dim = w.out_dim; m.in_dim = w.in_dim;
        return m;
    };
    std::vector<FusedLayerIn> in((size_t)n_layers);
    for (int l = 0; l < n_layers; ++l) {
        const LayerDev& L = s.layers[l];
        in[l].m[F_QKV] = mat(L.wqkv); in[l].m[F_WO] = mat(L.wo); in[l].m[F_W1] = mat(L.w1); in[l].m[F_W2] = mat(L.w2);
        in[l].gamma = L.gamma; in[l].kc = L.kc; in[l].vc = L.vc;
    }
    const bool first = s.gidx == 0, last = s.gidx == c.n_stages - 1;
    const FusedMatrix emb = mat(s.emb), unemb = mat(s.unemb);
    FusedCreate a;
    std::memset(&a, 0, sizeof(a));
    a.H = c.hidden; a.I = c.inter; a.heads = c.heads; a.vocab = c.vocab; a.n_layers = n_layers; a.eps = c.eps; a.max_pos = c.max_pos;
    a.n_ranks = n_ranks; a.rank = rank; a.sm_count = ws->sm_count; a.device = s.device;
    a.attn_split_min = c.attn_split_min > 0 ? c.attn_split_min : 32;
    a.no_cluster = c.cluster == 0;
    a.layers = in.data();
    a.emb = first ? &emb : nullptr;
    a.unemb = last ? &unemb : nullptr;
    a.gamma_final = s.layers.back().gamma;
    a.hidden = s.hidden; a.d_pos = s.d_pos; a.d_token = s.d_token; a.d_skip = first ? s.d_skip : nullptr; a.d_prompt = s.d_prompt;
    a.d_gen = s.d_gen; a.cos_t = s.cos_t; a.sin_t = s.sin_t; a.logits16 = s.logits16; a.logits32 = s.logits32; a.err = ws->err;
    a.stream = s.stream;
    QW3_CUDA(cudaSetDevice(s.device));
    // row-split: a rank computes only its blocks of the logits; the others stay NaN in the fp32 copy (test hook)
    if (tp && s.logits32) QW3_CUDA(cudaMemset(s.logits32, 0xff, (size_t)c.vocab * 4));
    return fused_create(a, &s.fused);
}

static int create_impl(const char* weight_dir, qw3_engine* e) {
    Qw3Config& c = e->cfg;
    QW3_TRY(validate_config(c));
    const bool tp = c.tensor_parallel != 0 && c.world > 1;   // one process per GPU, every matrix row-split: this handle runs all layers on its share
    const bool mp = c.world > 1 && !tp;                       // one process per GPU, layer pipeline: this handle owns stage `rank` only
    QW3_REQUIRE(!mp || c.n_stages == c.world, "qw3_create: with world > 1 the number of stages must equal world");
    QW3_REQUIRE(!tp || (c.n_stages == 1 && c.persistent >= 2), "qw3_create: tensor_parallel needs n_stages = 1 and persistent = 2");
    int ndev = 0;
    QW3_CUDA(cudaGetDeviceCount(&ndev));
    for (int s = 0; s < c.n_stages; ++s) {
        if (mp && s != c.rank) continue;
        if (c.device[s] < 0 || c.device[s] >= ndev) {   // Inference.cu:566-569
            set_last_error("stage %d wants device %d but only %d device(s) are visible", s, c.device[s], ndev);
            return QW3_ERR_DEVICE;
        }
    }
    const std::string dir(weight_dir);
    const int H = c.hidden, I = c.inter, V = c.vocab, N = mp ? 1 : c.n_stages;   // N: stages in this process
    e->st.resize(N);
    // initMultiGPU (Inference.cu:563-596): peer access between every pair of devices in use.
    for (int a = 0; a < N && !mp; ++a)
        for (int b = 0; b < N; ++b) {
            const int da = c.device[a], db = c.device[b];
            if (da == db) continue;
            int can = 0;
            QW3_CUDA(cudaDeviceCanAccessPeer(&can, da, db));
            if (!can) {
                set_last_error("P2P not supported between device %d and device %d", da, db);
                return QW3_ERR_DEVICE;
            }
            QW3_CUDA(cudaSetDevice(da));
            cudaError_t pe = cudaDeviceEnablePeerAccess(db, 0);
            if (pe == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else QW3_CUDA(pe);
        }
    std::vector<uint16_t> h_cos((size_t)c.max_pos * 64), h_sin((size_t)c.max_pos * 64);
    for (int pos = 0; pos < c.max_pos; ++pos)           // Inference.cu:444-454 (fp16 tables, host libm)
        for (int i = 0; i < 64; ++i) {
            const float inv_freq = 1.0f / powf(c.rope_base, float(2 * i) / float(c.head_dim));
            const float angle = float(pos) * inv_freq;
            const __half hc = __float2half_rn(cosf(angle)), hs = __float2half_rn(sinf(angle));
            std::memcpy(&h_cos[(size_t)pos * 64 + i], &hc, 2);
            std::memcpy(&h_sin[(size_t)pos * 64 + i], &hs, 2);
        }
    for (int si = 0; si < N; ++si) {
        Stage& s = e->st[si];
        s.gidx = mp ? c.rank : si;
        s.device = c.device[s.gidx]; s.l0 = c.first_layer[s.gidx]; s.l1 = c.first_layer[s.gidx + 1];
        QW3_CUDA(cudaSetDevice(s.device));
        QW3_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
        QW3_CUDA(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
        QW3_CUDA(cudaEventCreateWithFlags(&s.taken, cudaEventDisableTiming));
        QW3_TRY(qw3_ws_create(&s.ws));
        qw3_ws_set_pdl(s.ws, c.use_pdl);
        QW3_TRY(dev_alloc(e, s.device, &s.hidden, (size_t)H * 2));
        QW3_TRY(dev_alloc(e, s.device, &s.q, (size_t)H * 2));
        QW3_TRY(dev_alloc(e, s.device, &s.ctx, (size_t)H * 2));
        QW3_TRY(dev_alloc(e, s.device, &s.mlp, (size_t)I * 2));
        QW3_TRY(dev_alloc(e, s.device, &s.cos_t, h_cos.size() * 2));
        QW3_TRY(dev_alloc(e, s.device, &s.sin_t, h_sin.size() * 2));
        QW3_CUDA(cudaMemcpyAsync(s.cos_t, h_cos.data(), h_cos.size() * 2, cudaMemcpyHostToDevice, s.stream));
        QW3_CUDA(cudaMemcpyAsync(s.sin_t, h_sin.data(), h_sin.size() * 2, cudaMemcpyHostToDevice, s.stream));
        void* ints = nullptr;
        QW3_TRY(dev_alloc(e, s.device, &ints, 256));
        QW3_CUDA(cudaMemsetAsync(ints, 0, 256, s.stream));
        s.d_pos = static_cast<int*>(ints); s.d_step = s.d_pos + 1; s.d_token = s.d_pos + 2; s.d_skip = s.d_pos + 3;
        s.d_gen = s.d_pos + 8;   // generation counter of the sequence (part of the tags of the fused pass and of the chained stages)
        QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_prompt), (size_t)c.max_pos * 4));
        QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_out_ids), (size_t)c.max_pos * 4));
        QW3_CUDA(cudaMemsetAsync(s.hidden, 0, (size_t)H * 2, s.stream));
        s.layers.resize(s.l1 - s.l0);
        const size_t kv_bytes = (size_t)c.heads * c.max_pos * c.head_dim * 2;   // Inference.cu:676
        for (int l = s.l0; l < s.l1; ++l) {
            LayerDev& L = s.layers[l - s.l0];
            const std::string p = dir + "/layer_" + std::to_string(l) + "_";
            QW3_TRY(load_w4(e, s, L.wqkv, 3 * (int64_t)H, H, p + "wqkv.bin", p + "bqkv_scale.bin", p + "bqkv_zp.bin", true));
            QW3_TRY(load_w4(e, s, L.wo, H, H, p + "wo.bin", p + "wo_scale.bin", p + "wo_zp.bin", true));
            QW3_TRY(load_w4(e, s, L.w1, I, H, p + "w1.bin", p + "w1_scale.bin", p + "w1_zp.bin", true));
            QW3_TRY(load_w4(e, s, L.w2, H, I, p + "w2.bin", p + "w2_scale.bin", p + "w2_zp.bin", true));
            QW3_TRY(dev_alloc(e, s.device, &L.gamma, (size_t)H * 2));
            QW3_TRY(read_to_device(e, dir + "/rms_norm_gamma_" + std::to_string(l) + ".bin", L.gamma, (size_t)H * 2, s.stream));
            QW3_TRY(dev_alloc(e, s.device, &L.kc, kv_bytes));
            QW3_TRY(dev_alloc(e, s.device, &L.vc, kv_bytes));
            QW3_CUDA(cudaMemsetAsync(L.kc, 0, kv_bytes, s.stream));             // Inference.cu:431-437
            QW3_CUDA(cudaMemsetAsync(L.vc, 0, kv_bytes, s.stream));
        }
        if (s.gidx == 0)
            QW3_TRY(load_w4(e, s, s.emb, H, V, dir + "/word_embedding.bin", dir + "/word_embed_scale.bin",
                            dir + "/word_embed_zp.bin", false));
        if (s.gidx == c.n_stages - 1) {
            QW3_TRY(load_w4(e, s, s.unemb, V, H, dir + "/unembed.bin", dir + "/unembed_scale.bin", dir + "/unembed_zp.bin", true));
            QW3_TRY(dev_alloc(e, s.device, &s.logits16, (size_t)V * 2));
            if (c.keep_logits) QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.logits32), (size_t)V * 4));
        }
        QW3_CUDA(cudaStreamSynchronize(s.stream));
    }
    if (c.persistent >= 2) {
        for (int si = 0; si < N; ++si) QW3_TRY(create_fused(e, e->st[si]));
        if (tp && !e->st[0].fused) {
            set_last_error("tensor_parallel needs the fused pass");
            return QW3_ERR_ARG;
        }
    }
    if (c.persistent) {
        for (int si = 0; si < N; ++si) {
            Stage& s = e->st[si];
            if (s.fused) continue;
            bool ok = c.heads <= WS_ATT_MAX_HEADS;
            for (LayerDev& L : s.layers)
                ok = ok && pass_supports(w4_desc(L.wqkv.desc)) && pass_supports(w4_desc(L.wo.desc)) &&
                     pass_supports(w4_desc(L.w1.desc)) && pass_supports(w4_desc(L.w2.desc));
            if (s.gidx == c.n_stages - 1) ok = ok && pass_supports(w4_desc(s.unemb.desc));
            if (!ok) continue;   // shapes outside the persistent kernel's limits: per-operator launches
            QW3_CUDA(cudaSetDevice(s.device));
            QW3_TRY(pass_init_device());
            {   // tagged activations: 8 bytes per pair of halves
                const size_t hb = (size_t)c.hidden * 4, ib = (size_t)c.inter * 4;
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.hidden_t), hb));
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.ctx_t), hb));
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.mlp_t), ib));
                QW3_CUDA(cudaMemset(s.hidden_t, 0, hb));
                QW3_CUDA(cudaMemset(s.ctx_t, 0, hb));
                QW3_CUDA(cudaMemset(s.mlp_t, 0, ib));
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.qkv_t), 3 * hb));
                QW3_CUDA(cudaMemset(s.qkv_t, 0, 3 * hb));
            }
            QW3_TRY(build_pass_program(e, si, false, &s.ops_prompt, &s.n_ops_prompt));
            QW3_TRY(build_pass_program(e, si, true, &s.ops_decode, &s.n_ops_decode));
            {
                const int n_max = s.n_ops_decode > s.n_ops_prompt ? s.n_ops_decode : s.n_ops_prompt;
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_done), (size_t)(n_max + 64) * sizeof(int)));
                QW3_CUDA(cudaMemset(s.d_done, 0, (size_t)(n_max + 64) * sizeof(int)));
                s.d_epoch = s.d_done + n_max + 32;
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_tok_out_slot), 16));
                QW3_CUDA(cudaMemset(s.d_tok_out_slot, 0, 16));
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_xchg), pass_xchg_bytes()));
                QW3_CUDA(cudaMemset(s.d_xchg, 0, pass_xchg_bytes()));
            }
#ifdef QW3_TRACE
            {
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_trace), (size_t)(s.n_ops_decode + 1) * 8));
                QW3_CUDA(cudaMemset(s.d_trace, 0, (size_t)(s.n_ops_decode + 1) * 8));
                const size_t t2 = (size_t)256 * s.n_ops_decode * 8 * 8;
                QW3_TRY(dev_alloc(e, s.device, reinterpret_cast<void**>(&s.d_trace2), t2));
                QW3_CUDA(cudaMemset(s.d_trace2, 0, t2));
            }
#endif
            s.persistent = true;
        }
    }
    if (mp) {
        Stage& s = e->st[0];
        QW3_TRY(dev_alloc(e, s.device, &e->mailbox, mailbox_bytes(H)));
        QW3_CUDA(cudaMemset(e->mailbox, 0, mailbox_bytes(H)));
    }
    QW3_CUDA(cudaSetDevice(e->st[0].device));
    QW3_CUDA(cudaEventCreate(&e->ev0));
    QW3_CUDA(cudaEventCreate(&e->ev1));
    QW3_CUDA(cudaEventCreate(&e->ev2));
    if (e->pinned) {
        cudaFreeHost(e->pinned);
        e->pinned = nullptr;
        e->pinned_bytes = 0;
    }
    if (c.use_graph && !tp) {   // row-split: captured in qw3_tp_connect, once the peers' buffers are known
        for (int si = 0; si < N; ++si) {
            QW3_TRY(capture_stage_graph(e, si, false, &e->st[si].g_prompt, &e->st[si].launches_prompt));
            QW3_TRY(capture_stage_graph(e, si, true, &e->st[si].g_decode, &e->st[si].launches_decode));
        }
    }
    return QW3_OK;
}

int qw3_create(const char* weight_dir, const Qw3Config* cfg, qw3_handle* out) {
    QW3_REQUIRE(weight_dir && out, "qw3_create: null pointer");
    qw3_engine* e = new (std::nothrow) qw3_engine();
    if (!e) return QW3_ERR_NOMEM;
    if (cfg) e->cfg = *cfg; else qw3_config_default(&e->cfg);
    int rc = create_impl(weight_dir, e);
    if (rc != QW3_OK) {
        qw3_destroy(e);
        return rc;
    }
    *out = e;
    return QW3_OK;
}

// ---- one process per GPU: this process drives stage `rank`; neighbours are reached through mailboxes ----
static int pass_mp(qw3_engine* e, bool decode, bool layers) {
    Stage& s = e->st[0];
    QW3_CUDA(cudaSetDevice(s.device));
    const bool linked = decode && layers && e->linked_now;
    cudaGraphExec_t g = linked ? s.g_linked : (decode ? s.g_decode : s.g_prompt);
    if (layers && g) {
        QW3_CUDA(cudaGraphLaunch(g, s.stream));
        e->launches += linked ? s.launches_linked : (decode ? s.launches_decode : s.launches_prompt);
    } else {
        int n = 0;
        QW3_TRY(enqueue_stage_pass(e, 0, decode, layers, false, &n));
        e->launches += n;
    }
    return QW3_OK;
}
static int mp_send(qw3_engine* e) {
    Stage& s = e->st[0];
    e->launches += 1;
    return handoff_send(s.hidden, e->next_mb, e->mailbox, ++e->msg_out, e->cfg.hidden, ws_struct(s.ws)->err, s.stream);
}
static int mp_recv(qw3_engine* e) {
    Stage& s = e->st[0];
    e->launches += 1;
    return handoff_recv(s.hidden, e->mailbox, e->prev_mb, ++e->msg_in, e->cfg.hidden, ws_struct(s.ws)->err, s.stream);
}

static int decode_loop_mp(qw3_engine* e, int max_new, int32_t* out_ids, int32_t* n_out) {
    const Qw3Config& c = e->cfg;
    Stage& s = e->st[0];
    const bool first = s.gidx == 0, last = s.gidx == c.n_stages - 1;
    if (!e->next_mb || !e->prev_mb) {
        set_last_error("one process per GPU: call qw3_stage_connect before generating");
        return QW3_ERR_STATE;
    }
    QW3_CUDA(cudaSetDevice(s.device));
    if (last) QW3_CUDA(cudaMemsetAsync(s.d_step, 0, 4, s.stream));
    for (int step = 0; step < max_new; ++step) {
        const bool very_first = (e->sampled == 0);
        const bool layers = !(c.sample_first && very_first);
        // From the second pass through the layers on, the stages are chained inside the token-pass kernels: the last
        // operator of a stage stores the tagged hidden state into the next GPU's inbox, the first operator of the next
        // stage polls it, and the sampled id reaches the first stage the same way.  Every stage takes this decision
        // from the same counters, so the stages switch at the same step.
        const bool chained = layers && e->chain_decode && s.ops_linked != nullptr && e->sampled >= (c.sample_first ? 2 : 1);
        if (chained) {
            e->linked_now = true;
            const int rc = pass_mp(e, true, true);
            e->linked_now = false;
            QW3_TRY(rc);
            e->seq_len += 1;
        } else if (layers) {
            if (very_first) {
                // Reference flow (Inference.cu:1357): the last stage's final hidden state re-enters layer 0.
                if (last) QW3_TRY(mp_send(e));
                if (first) {
                    QW3_TRY(mp_recv(e));
                    const int one = 1;
                    QW3_CUDA(cudaMemcpyAsync(s.d_skip, &one, 4, cudaMemcpyHostToDevice, s.stream));
                }
            } else {
                if (last) { QW3_TRY(token_send(s.d_token, e->next_mb, ++e->tok_out, s.stream)); e->launches += 1; }
                if (first) { QW3_TRY(token_recv(s.d_token, e->mailbox, ++e->tok_in, ws_struct(s.ws)->err, s.stream)); e->launches += 1; }
            }
            if (!first) QW3_TRY(mp_recv(e));
            QW3_TRY(pass_mp(e, true, true));
            if (!last) QW3_TRY(mp_send(e));
            e->seq_len += 1;
        } else if (last) {
            QW3_TRY(pass_mp(e, true, false));   // sample-only pass on the last stage
        }
        e->sampled += 1;
    }
    QW3_CUDA(cudaEventRecord(e->ev2, s.stream));
    QW3_CUDA(cudaStreamSynchronize(s.stream));
    if (last && max_new > 0) QW3_CUDA(cudaMemcpy(out_ids, s.d_out_ids, (size_t)max_new * 4, cudaMemcpyDeviceToHost));
    if (n_out) *n_out = last ? max_new : 0;     // the ids come out of the last stage's process
    QW3_CUDA(cudaEventElapsedTime(&e->decode_ms, e->ev1, e->ev2));
    return qw3_ws_check(s.ws, s.stream);
}

static int generate_mp(qw3_engine* e, const int32_t* prompt, int32_t n_prompt, int32_t max_new, int32_t* out_ids, int32_t* n_out) {
    const Qw3Config& c = e->cfg;
    Stage& s = e->st[0];
    const bool first = s.gidx == 0, last = s.gidx == c.n_stages - 1;
    if (!e->next_mb || !e->prev_mb) {
        set_last_error("one process per GPU: call qw3_stage_connect before generating");
        return QW3_ERR_STATE;
    }
    e->launches = 0;
    QW3_CUDA(cudaSetDevice(s.device));
    QW3_CUDA(cudaMemsetAsync(s.d_pos, 0, 16, s.stream));
    e->gen += 1;   // every stage counts the generations alike: the cross-GPU tags of this sequence
    if (s.d_gen) QW3_CUDA(cudaMemcpyAsync(s.d_gen, &e->gen, 4, cudaMemcpyHostToDevice, s.stream));
    if (first) QW3_CUDA(cudaMemcpyAsync(s.d_prompt, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s.stream));
    QW3_CUDA(cudaEventRecord(e->ev0, s.stream));
    if (use_batched_prefill(e, n_prompt)) {
        for (int t0 = 0; t0 < n_prompt; t0 += PF_BLOCK)
            QW3_TRY(prefill_block_mp(e, t0, n_prompt - t0 < PF_BLOCK ? n_prompt - t0 : PF_BLOCK));
    } else {
        for (int t = 0; t < n_prompt; ++t) {     // stages overlap on successive prompt tokens (two inbox slots)
            if (!first) QW3_TRY(mp_recv(e));
            QW3_TRY(pass_mp(e, false, true));
            if (!last) QW3_TRY(mp_send(e));
        }
    }
    QW3_CUDA(cudaEventRecord(e->ev1, s.stream));
    e->seq_len = n_prompt;
    e->sampled = 0;
    QW3_TRY(decode_loop_mp(e, max_new, out_ids, n_out));
    QW3_CUDA(cudaEventElapsedTime(&e->prompt_ms, e->ev0, e->ev1));
    return QW3_OK;
}

// The decode loop of generateResponse (Inference.cu:1352-1405), continuing from the current
// sequence state; max_new ids are read back at the end (the host never waits inside the loop).
static int decode_loop(qw3_engine* e, int max_new, int32_t* out_ids) {
    const Qw3Config& c = e->cfg;
    const int N = c.n_stages;
    Stage &s0 = e->st[0], &sl = e->st[N - 1];
    QW3_CUDA(cudaSetDevice(sl.device));
    QW3_CUDA(cudaMemsetAsync(sl.d_step, 0, 4, sl.stream));
    for (int step = 0; step < max_new; ++step) {
        const bool very_first = (e->sampled == 0);
        bool layers = true;
        if (c.sample_first && very_first) layers = false;
        if (layers) {
            if (very_first) {
                // Reference flow: step 0 re-enters layer 0 with the final hidden state of the last
                // prompt token (Inference.cu:1357): move it back to stage 0 and skip the gather.
                if (N > 1) QW3_TRY(handoff(e, N - 1, 0, true, false));
                const int one = 1;
                QW3_CUDA(cudaSetDevice(s0.device));
                QW3_CUDA(cudaMemcpyAsync(s0.d_skip, &one, 4, cudaMemcpyHostToDevice, s0.stream));
            } else if (N > 1) {
                QW3_TRY(handoff(e, N - 1, 0, false, true));                           // sampled id -> stage 0
            }
        }
        QW3_TRY(run_pass(e, true, layers));
        if (layers) e->seq_len += 1;
        e->sampled += 1;
    }
    QW3_CUDA(cudaSetDevice(s0.device));
    QW3_CUDA(cudaStreamWaitEvent(s0.stream, sl.done, 0));
    QW3_CUDA(cudaEventRecord(e->ev2, s0.stream));
    QW3_CUDA(cudaStreamSynchronize(s0.stream));
    QW3_CUDA(cudaSetDevice(sl.device));
    QW3_CUDA(cudaStreamSynchronize(sl.stream));
    if (max_new > 0) QW3_CUDA(cudaMemcpy(out_ids, sl.d_out_ids, (size_t)max_new * 4, cudaMemcpyDeviceToHost));
    QW3_CUDA(cudaEventElapsedTime(&e->decode_ms, e->ev1, e->ev2));
    for (int si = 0; si < N; ++si) {
        QW3_CUDA(cudaSetDevice(e->st[si].device));
        QW3_TRY(qw3_ws_check(e->st[si].ws, e->st[si].stream));
    }
    return QW3_OK;
}

int qw3_generate(qw3_handle e, const int32_t* prompt, int32_t n_prompt, int32_t max_new, int32_t* out_ids, int32_t* n_out) {
    QW3_REQUIRE(e && prompt && (out_ids || max_new == 0), "qw3_generate: null pointer");
    const Qw3Config& c = e->cfg;
    if (n_prompt < 1 || max_new < 0 || (int64_t)n_prompt + max_new > c.max_pos) {   // Inference.cu:1301, plus the new tokens
        set_last_error("qw3_generate: prompt of %d plus %d new tokens does not fit max_pos=%d", n_prompt, max_new, c.max_pos);
        return QW3_ERR_RANGE;
    }
    for (int t = 0; t < n_prompt; ++t)
        if (prompt[t] < 0 || prompt[t] >= c.vocab) {
            set_last_error("qw3_generate: token id %d at %d is outside [0, %d)", prompt[t], t, c.vocab);
            return QW3_ERR_RANGE;
        }
    const bool tp = c.tensor_parallel != 0 && c.world > 1;
    if (tp && !e->tp_connected) {
        set_last_error("tensor_parallel: call qw3_tp_connect before generating");
        return QW3_ERR_STATE;
    }
    if (c.world > 1 && !tp) return generate_mp(e, prompt, n_prompt, max_new, out_ids, n_out);
    const int N = c.n_stages;
    Stage &s0 = e->st[0], &sl = e->st[N - 1];
    e->launches = 0;
    e->seq_len = 0;
    // The object is reusable: position and step restart for every call; the generation counter goes into the tags
    // of the words the fused pass exchanges, so that words of an earlier sequence are never taken for this one's.
    e->gen += 1;
    for (int si = 0; si < N; ++si) {
        Stage& s = e->st[si];
        QW3_CUDA(cudaSetDevice(s.device));
        QW3_CUDA(cudaMemsetAsync(s.d_pos, 0, 16, s.stream));
        QW3_CUDA(cudaMemcpyAsync(s.d_gen, &e->gen, 4, cudaMemcpyHostToDevice, s.stream));
    }
    QW3_CUDA(cudaSetDevice(s0.device));
    QW3_CUDA(cudaMemcpyAsync(s0.d_prompt, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s0.stream));
    QW3_CUDA(cudaEventRecord(e->ev0, s0.stream));
    if (use_batched_prefill(e, n_prompt)) {
        for (int t0 = 0; t0 < n_prompt; t0 += PF_BLOCK) QW3_TRY(prefill_block(e, t0, n_prompt - t0 < PF_BLOCK ? n_prompt - t0 : PF_BLOCK));
    } else {
        for (int t = 0; t < n_prompt; ++t) QW3_TRY(run_pass(e, false, true));        // Inference.cu:1304-1343
    }
    QW3_CUDA(cudaSetDevice(s0.device));
    QW3_CUDA(cudaStreamWaitEvent(s0.stream, sl.done, 0));
    QW3_CUDA(cudaEventRecord(e->ev1, s0.stream));
    e->seq_len = n_prompt;
    e->sampled = 0;
    QW3_TRY(decode_loop(e, max_new, out_ids));
    if (n_out) *n_out = max_new;
    QW3_CUDA(cudaEventElapsedTime(&e->prompt_ms, e->ev0, e->ev1));
    return QW3_OK;
}

int qw3_decode_more(qw3_handle e, int32_t max_new, int32_t* out_ids, int32_t* n_out) {
    QW3_REQUIRE(e && (out_ids || max_new == 0), "qw3_decode_more: null pointer");
    if (e->seq_len < 1 || e->sampled < 1) {
        set_last_error("qw3_decode_more: nothing to continue; call qw3_generate with max_new >= 1 first");
        return QW3_ERR_STATE;
    }
    if (max_new < 0 || (int64_t)e->seq_len + max_new > e->cfg.max_pos) {
        set_last_error("qw3_decode_more: %d more tokens after %d do not fit max_pos=%d", max_new, e->seq_len, e->cfg.max_pos);
        return QW3_ERR_RANGE;
    }
    Stage& s0 = e->st[0];
    e->launches = 0;
    e->prompt_ms = 0.f;
    QW3_CUDA(cudaSetDevice(s0.device));
    QW3_CUDA(cudaEventRecord(e->ev1, s0.stream));
    if (e->cfg.world > 1 && !e->cfg.tensor_parallel) return decode_loop_mp(e, max_new, out_ids, n_out);
    QW3_TRY(decode_loop(e, max_new, out_ids));
    if (n_out) *n_out = max_new;
    return QW3_OK;
}

int qw3_last_logits(qw3_handle e, float* out_vocab) {
    QW3_REQUIRE(e && out_vocab, "qw3_last_logits: null pointer");
    Stage& sl = e->st.back();
    if (!sl.logits32) {
        set_last_error("qw3_last_logits: the handle was created with keep_logits = 0");
        return QW3_ERR_STATE;
    }
    QW3_CUDA(cudaSetDevice(sl.device));
    QW3_CUDA(cudaStreamSynchronize(sl.stream));
    QW3_CUDA(cudaMemcpy(out_vocab, sl.logits32, (size_t)e->cfg.vocab * 4, cudaMemcpyDeviceToHost));
    return QW3_OK;
}

int qw3_set_batched_prefill(qw3_handle e, int on) {
    QW3_REQUIRE(e, "qw3_set_batched_prefill: null handle");
    e->batched_prefill = on < 0 ? -1 : (on != 0);   // one process per GPU: every stage must be set alike
    return QW3_OK;
}

int qw3_last_timing(qw3_handle e, float* prompt_ms, float* decode_ms) {
    QW3_REQUIRE(e, "qw3_last_timing: null handle");
    if (prompt_ms) *prompt_ms = e->prompt_ms;
    if (decode_ms) *decode_ms = e->decode_ms;
    return QW3_OK;
}

int qw3_last_launches(qw3_handle e, int64_t* n) {
    QW3_REQUIRE(e && n, "qw3_last_launches: null pointer");
    *n = e->launches;
    return QW3_OK;
}

static Stage* stage_of_layer(qw3_engine* e, int layer) {
    for (Stage& s : e->st)
        if (layer >= s.l0 && layer < s.l1) return &s;
    return nullptr;
}

int qw3_kv_upload(qw3_handle e, int32_t layer, int32_t which, const void* host_f16, int64_t upto) {
    QW3_REQUIRE(e && host_f16, "qw3_kv_upload: null pointer");
    Stage* s = stage_of_layer(e, layer);
    QW3_REQUIRE(s && upto >= 0 && upto <= e->cfg.max_pos, "qw3_kv_upload: layer or row count out of range");
    const Qw3Config& c = e->cfg;
    LayerDev& L = s->layers[layer - s->l0];
    QW3_CUDA(cudaSetDevice(s->device));
    __half* dst = static_cast<__half*>(which ? L.vc : L.kc);
    const __half* src = static_cast<const __half*>(host_f16);
    for (int h = 0; h < c.heads; ++h)
        QW3_CUDA(cudaMemcpyAsync(dst + (size_t)h * c.max_pos * 128, src + (size_t)h * upto * 128, (size_t)upto * 256,
                                 cudaMemcpyHostToDevice, s->stream));
    QW3_CUDA(cudaStreamSynchronize(s->stream));
    return QW3_OK;
}

int qw3_layer_decode(qw3_handle e, int32_t layer, int32_t pos, void* host_hidden) {
    QW3_REQUIRE(e && host_hidden, "qw3_layer_decode: null pointer");
    Stage* s = stage_of_layer(e, layer);
    QW3_REQUIRE(s && pos >= 0 && pos < e->cfg.max_pos, "qw3_layer_decode: layer or pos out of range");
    QW3_CUDA(cudaSetDevice(s->device));
    QW3_CUDA(cudaMemcpyAsync(s->hidden, host_hidden, (size_t)e->cfg.hidden * 2, cudaMemcpyHostToDevice, s->stream));
    QW3_CUDA(cudaMemcpyAsync(s->d_pos, &pos, 4, cudaMemcpyHostToDevice, s->stream));
    int n = 0;
    QW3_TRY(enqueue_layer(e, *s, layer - s->l0, false, &n));
    QW3_CUDA(cudaMemcpyAsync(host_hidden, s->hidden, (size_t)e->cfg.hidden * 2, cudaMemcpyDeviceToHost, s->stream));
    QW3_CUDA(cudaStreamSynchronize(s->stream));
    return qw3_ws_check(s->ws, s->stream);
}

int qw3_stage_hidden(qw3_handle e, int32_t stage, void* host_hidden) {
    QW3_REQUIRE(e && host_hidden && stage >= 0 && stage < (int)e->st.size(), "qw3_stage_hidden: bad argument");
    Stage& s = e->st[stage];
    QW3_CUDA(cudaSetDevice(s.device));
    QW3_CUDA(cudaStreamSynchronize(s.stream));
    QW3_CUDA(cudaMemcpy(host_hidden, s.hidden, (size_t)e->cfg.hidden * 2, cudaMemcpyDeviceToHost));
    return QW3_OK;
}

#ifdef QW3_TRACE
int qw3_debug_trace(qw3_handle e, int32_t stage, uint64_t* out, int32_t max_entries, int32_t* n_entries) {
    QW3_REQUIRE(e && out && n_entries && stage >= 0 && stage < (int)e->st.size(), "qw3_debug_trace: bad argument");
    Stage& s = e->st[stage];
    if (s.fused) {   // fused pass, tracing build: the raw stamps [grid][n_layers][16]; *n_entries = values copied
        size_t bytes = 0;
        const void* tr = fused_trace(s.fused, &bytes);
        if (!tr) {
            set_last_error("qw3_debug_trace: the library was not built with -DQW3_TRACE");
            return QW3_ERR_STATE;
        }
        QW3_CUDA(cudaSetDevice(s.device));
        QW3_CUDA(cudaStreamSynchronize(s.stream));
        const size_t want = (size_t)(max_entries < 0 ? -max_entries : max_entries) * 8;
        const size_t m = want < bytes ? want : bytes;
        QW3_CUDA(cudaMemcpy(out, tr, m, cudaMemcpyDeviceToHost));
        *n_entries = (int32_t)(m / 8);
        return QW3_OK;
    }
    if (!s.d_trace) {
        set_last_error("qw3_debug_trace: the stage runs neither pass kernel");
        return QW3_ERR_STATE;
    }
    QW3_CUDA(cudaSetDevice(s.device));
    QW3_CUDA(cudaStreamSynchronize(s.stream));
    if (max_entries < 0) {   // detailed form: -max_entries values of [grid][n_ops][8] per-CTA event times
        const size_t total = (size_t)256 * s.n_ops_decode * 8;
        const size_t m = (size_t)(-max_entries) < total ? (size_t)(-max_entries) : total;
        QW3_CUDA(cudaMemcpy(out, s.d_trace2, m * 8, cudaMemcpyDeviceToHost));
        *n_entries = s.n_ops_decode;
        return QW3_OK;
    }
    const int n = s.n_ops_decode + 1 < max_entries ? s.n_ops_decode + 1 : max_entries;
    QW3_CUDA(cudaMemcpy(out, s.d_trace, (size_t)n * 8, cudaMemcpyDeviceToHost));
    *n_entries = n;
    return QW3_OK;
}
#endif  // QW3_TRACE

int qw3_stage_layers(const Qw3Config* cfg, int32_t stage, int32_t* first, int32_t* count) {
    QW3_REQUIRE(cfg && first && count, "qw3_stage_layers: null pointer");
    Qw3Config c = *cfg;
    QW3_TRY(validate_config(c));
    QW3_REQUIRE(stage >= 0 && stage < c.n_stages, "qw3_stage_layers: stage out of range");
    *first = c.first_layer[stage];
    *count = c.first_layer[stage + 1] - c.first_layer[stage];
    return QW3_OK;
}

int qw3_stage_export(qw3_handle e, void* out_handle_64B) {
    QW3_REQUIRE(e && out_handle_64B, "qw3_stage_export: null pointer");
    if (!e->mailbox) {
        set_last_error("qw3_stage_export: the handle was not created with world > 1");
        return QW3_ERR_STATE;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
    cudaIpcMemHandle_t h;
    QW3_CUDA(cudaSetDevice(e->st[0].device));
    QW3_CUDA(cudaIpcGetMemHandle(&h, e->mailbox));
    std::memcpy(out_handle_64B, &h, 64);
    return QW3_OK;
}

int qw3_stage_connect(qw3_handle e, const void* next_stage_handle_64B, const void* prev_stage_handle_64B) {
    QW3_REQUIRE(e && next_stage_handle_64B && prev_stage_handle_64B, "qw3_stage_connect: null pointer");
    if (!e->mailbox || e->next_mb) {
        set_last_error("qw3_stage_connect: needs a handle created with world > 1 that is not connected yet");
        return QW3_ERR_STATE;
    }
    cudaIpcMemHandle_t hn, hp;
    std::memcpy(&hn, next_stage_handle_64B, 64);
    std::memcpy(&hp, prev_stage_handle_64B, 64);
    QW3_CUDA(cudaSetDevice(e->st[0].device));
    QW3_CUDA(cudaIpcOpenMemHandle(&e->next_mb, hn, cudaIpcMemLazyEnablePeerAccess));
    if (std::memcmp(&hn, &hp, 64) == 0) {   // two stages: the next stage is also the previous one
        e->prev_mb = e->next_mb;
        e->next_is_prev = true;
    } else {
        QW3_CUDA(cudaIpcOpenMemHandle(&e->prev_mb, hp, cudaIpcMemLazyEnablePeerAccess));
    }
    // Chained decode passes: their operator list names the neighbours' mailboxes, so it is built here.
    Stage& s = e->st[0];
    if (s.persistent) {
        const bool last = s.gidx == e->cfg.n_stages - 1;
        if (last) {   // the first stage is the next one in the ring
            unsigned long long* tw = static_cast<unsigned long long*>(mailbox_token_word(e->next_mb));
            QW3_CUDA(cudaMemcpy(s.d_tok_out_slot, &tw, sizeof(tw), cudaMemcpyHostToDevice));
        }
        QW3_TRY(build_pass_program(e, 0, true, &s.ops_linked, &s.n_ops_linked, true));
        if (e->cfg.use_graph) {
            e->linked_now = true;
            const int rc = capture_stage_graph(e, 0, true, &s.g_linked, &s.launches_linked);
            e->linked_now = false;
            QW3_TRY(rc);
        }
    }
    return QW3_OK;
}

int qw3_handoff_wait(const int32_t* d_flag, int32_t want, int64_t limit_clocks, int32_t code, qw3_ws_t ws, void* stream) {
    QW3_REQUIRE(d_flag && ws, "qw3_handoff_wait: null pointer");
    QW3_REQUIRE(limit_clocks > 0, "qw3_handoff_wait: the limit must be positive");
    return flag_wait_launch(d_flag, want, limit_clocks, ws_struct(ws)->err, code, static_cast<cudaStream_t>(stream));
}

int qw3_tp_export(qw3_handle e, void* out_handle_64B) {
    QW3_REQUIRE(e && out_handle_64B, "qw3_tp_export: null pointer");
    if (!(e->cfg.tensor_parallel && e->cfg.world > 1) || !e->st[0].fused) {
        set_last_error("qw3_tp_export: the handle was not created with tensor_parallel = 1 and world > 1");
        return QW3_ERR_STATE;
    }
    cudaIpcMemHandle_t h;
    QW3_CUDA(cudaSetDevice(e->st[0].device));
    QW3_CUDA(cudaIpcGetMemHandle(&h, fused_exchange_base(e->st[0].fused, nullptr)));
    std::memcpy(out_handle_64B, &h, 64);
    return QW3_OK;
}

int qw3_tp_connect(qw3_handle e, const void* handles_world_x_64B) {
    QW3_REQUIRE(e && handles_world_x_64B, "qw3_tp_connect: null pointer");
    if (!(e->cfg.tensor_parallel && e->cfg.world > 1) || !e->st[0].fused || e->tp_connected) {
        set_last_error("qw3_tp_connect: needs a handle created with tensor_parallel = 1 and world > 1 that is not connected yet");
        return QW3_ERR_STATE;
    }
    QW3_CUDA(cudaSetDevice(e->st[0].device));
    const uint8_t* hs = static_cast<const uint8_t*>(handles_world_x_64B);
    e->tp_peers.assign((size_t)e->cfg.world, nullptr);
    for (int r = 0; r < e->cfg.world; ++r) {
        if (r == e->cfg.rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, hs + 64 * (size_t)r, 64);
        QW3_CUDA(cudaIpcOpenMemHandle(&e->tp_peers[r], h, cudaIpcMemLazyEnablePeerAccess));
        fused_set_peer(e->st[0].fused, r, e->tp_peers[r]);
    }
    // The graphs captured at creation hold the launch parameters of that moment, without the peers' buffers:
    // capture them again now that every address is known.
    Stage& s = e->st[0];
    if (e->cfg.use_graph) {
        if (s.g_prompt) { cudaGraphExecDestroy(s.g_prompt); s.g_prompt = nullptr; }
        if (s.g_decode) { cudaGraphExecDestroy(s.g_decode); s.g_decode = nullptr; }
        QW3_TRY(capture_stage_graph(e, 0, false, &s.g_prompt, &s.launches_prompt));
        QW3_TRY(capture_stage_graph(e, 0, true, &s.g_decode, &s.launches_decode));
    }
    e->tp_connected = true;
    return QW3_OK;
}

int qw3_set_chained_decode(qw3_handle e, int on) {
    QW3_REQUIRE(e, "qw3_set_chained_decode: null handle");
    e->chain_decode = on != 0;
    return QW3_OK;
}

}  // extern "C"
