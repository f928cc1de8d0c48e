// Small operators of the decode path on sm_100a: the bit-exact materialising dequantisation
// (test hook), RMSNorm, RoPE + KV append, split-KV decode attention, the packed embedding gather
// and the device arg-max.  Each cites the reference kernel it replaces.
#include "common.cuh"

namespace qw3 {

const Workspace* ws_struct(qw3_ws_t ws);
bool ws_pdl(qw3_ws_t ws);

// Launch helper: optional programmatic dependent launch attribute.
template <typename... KArgs, typename... Args>
static cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- dequantAwqKernel (Inference.cu:76-106): one thread per packed byte ------------------------
__global__ void dequant_w4_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scale,
                                  const __half* __restrict__ zp, long long n_alloc, long long rows, long long cols,
                                  __half* __restrict__ out) {
    const long long pc = (cols + 1) / 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * pc) return;
    const long long r = idx / pc, b = idx - r * pc, c = 2 * b;
    const uint32_t byte = packed[idx];
    const long long g = (c / 128) % n_alloc;  // c and c+1 share a group (128 is even)
    const __half z = zp[g], s = scale[g];
    out[r * cols + c] = dequant_one(byte & 15u, z, s);
    if (c + 1 < cols) out[r * cols + c + 1] = dequant_one(byte >> 4, z, s);
}

// ---- rmsNormKernel (Inference.cu:111-145) ------------------------------------------------------------
__global__ void __launch_bounds__(512) rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma,
                                                      int n, float eps, __half* __restrict__ out) {
    __shared__ double dsum[16];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double s = 0.0;
    for (int j = tid; j < n; j += 512) {
        const float v = __half2float(x[j]);
        s += (double)(v * v);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) s += shfl_xor_double(s, m);
    if (lane == 0) dsum[warp] = s;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int w = 0; w < 16; ++w) tot += dsum[w];
    const float mean_sq = __fdiv_rn((float)tot, (float)n);
    const __half sc = __float2half_rn(__fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps))));
    for (int j = tid; j < n; j += 512) out[j] = h_mul(h_mul(x[j], sc), gamma[j]);
}

// ---- QKV split + applyRotaryKernel + KV append (Inference.cu:1070-1103, 150-177) -------------------
__global__ void rope_kv_kernel(const __half* __restrict__ qkv, __half* __restrict__ q_out, __half* __restrict__ kc,
                               __half* __restrict__ vc, const __half* __restrict__ cos_t, const __half* __restrict__ sin_t,
                               int hidden, long long max_pos, const int* __restrict__ d_pos, int pos_imm) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;  // pair of adjacent elements
    if (pair >= 3 * hidden / 2) return;
    const int pos = d_pos ? *d_pos : pos_imm;
    const int i = 2 * pair, sec = i / hidden, idx = i - sec * hidden, head = idx >> 7, d = idx & 127;
    const __half2 v = *reinterpret_cast<const __half2*>(qkv + i);
    __half o0 = __low2half(v), o1 = __high2half(v);
    if (sec < 2) {
        const __half cs = cos_t[(size_t)pos * 64 + (d >> 1)], sn = sin_t[(size_t)pos * 64 + (d >> 1)];
        const __half x0 = o0, x1 = o1;
        rope_pair(x0, x1, cs, sn, o0, o1);
    }
    __half* dst = sec == 0 ? q_out + idx : (sec == 1 ? kc : vc) + ((size_t)head * max_pos + pos) * 128 + d;
    *reinterpret_cast<__half2*>(dst) = __halves2half2(o0, o1);
}

// ---- gather lambda (Inference.cu:1310-1315) on the packed [hidden][vocab] matrix -----------------
// Token id = d_token[d_index ? *d_index : 0] when d_token is set, else tok_imm.  When *d_skip is
// non-zero the hidden state is left as it is (decode step 0 of the reference flow re-enters layer 0
// with the last prompt token's final hidden state, Inference.cu:1355-1363).
__global__ void embed_gather_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scale,
                                    const __half* __restrict__ zp, long long n_alloc, int hidden, long long vocab,
                                    const int* __restrict__ d_token, const int* __restrict__ d_index,
                                    const int* __restrict__ d_skip, int tok_imm, __half* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= hidden) return;
    if (d_skip && *d_skip) return;
    long long tok = d_token ? d_token[d_index ? *d_index : 0] : tok_imm;
    if (tok < 0 || tok >= vocab) tok = 0;  // ids are validated on the host; never index out of range
    const long long pc = (vocab + 1) / 2;
    const uint32_t byte = packed[(long long)idx * pc + (tok >> 1)];
    const uint32_t q = (tok & 1) ? (byte >> 4) : (byte & 15u);
    const long long g = (tok / 128) % n_alloc;
    out[idx] = dequant_one(q, zp[g], scale[g]);
}

// End of one token pass: publish the sampled id, advance the device-side position and step.
__global__ void step_tail_kernel(int* d_pos, int* d_step, const int* d_token, int* d_out_ids, int* d_skip, int* d_epoch) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    if (d_out_ids && d_token && d_step) {
        d_out_ids[*d_step] = *d_token;
        *d_step += 1;
    }
    if (d_pos) *d_pos += 1;
    if (d_skip) *d_skip = 0;
    if (d_epoch) *d_epoch += 1;   // the persistent pass before this kernel used epoch *d_epoch + 1
}

// ---- attentionKernel (Inference.cu:182-266), intended math, split over the KV length --------------
// grid (heads, splits), 128 threads.  A half-warp owns one cache row at a time (16 lanes x 8
// halves = 128 dims, one 16-byte load per lane) and keeps an online-softmax state; the 8 states of
// the CTA, then the `splits` CTAs of a head, are merged in a fixed order by the last to arrive.
constexpr int ATT_THREADS = 128;
constexpr int ATT_GROUPS = ATT_THREADS / 16;

__device__ __forceinline__ void att_merge(const float* st, int n, int stride, int i, float& M, float& L, float& O) {
    M = -INFINITY;
    for (int g = 0; g < n; ++g) M = fmaxf(M, st[g * stride + 128]);
    L = 0.0f;
    O = 0.0f;
    for (int g = 0; g < n; ++g) {
        const float m = st[g * stride + 128];
        const float w = (m == -INFINITY) ? 0.0f : expf(m - M);
        L += st[g * stride + 129] * w;
        O += st[g * stride + i] * w;
    }
}

__global__ void __launch_bounds__(ATT_THREADS)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ kc, const __half* __restrict__ vc,
                   long long max_pos, const int* __restrict__ d_pos, int pos_imm, __half* __restrict__ ctx,
                   float* att_part, int* att_count) {
    __shared__ float st[ATT_GROUPS * WS_ATT_STRIDE];
    __shared__ float mrg[WS_ATT_MAX_SPLITS * WS_ATT_STRIDE];
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, split = blockIdx.y, S = gridDim.y;
    const int tid = threadIdx.x, lane = tid & 31, grp = tid >> 4, sl = tid & 15;
    const int len = (d_pos ? *d_pos : pos_imm) + 1;   // rows 0..pos
    const int chunk = (len + S - 1) / S;
    const int p0 = split * chunk, p1 = min(len, p0 + chunk);

    float qf[8];
    {
        const uint4 qv = *reinterpret_cast<const uint4*>(q + head * 128 + sl * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            qf[2 * e] = f.x;
            qf[2 * e + 1] = f.y;
        }
    }
    const float scale = 1.0f / sqrtf(128.0f);                     // Inference.cu:218
    const __half* kh = kc + (size_t)head * max_pos * 128 + sl * 8;
    const __half* vh = vc + (size_t)head * max_pos * 128 + sl * 8;
    float m = -INFINITY, l = 0.0f, o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.0f;

    constexpr int UN = 4;
    for (int kb = p0; kb < p1; kb += ATT_GROUPS * UN) {   // trip count uniform across the CTA
        const int k0 = kb + grp;
        uint4 kv[UN], vv[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int k = k0 + u * ATT_GROUPS;
            if (k < p1) {
                kv[u] = *reinterpret_cast<const uint4*>(kh + (size_t)k * 128);
                vv[u] = *reinterpret_cast<const uint4*>(vh + (size_t)k * 128);
            } else {
                kv[u] = make_uint4(0, 0, 0, 0);
                vv[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int k = k0 + u * ATT_GROUPS;   // uniform within the half-warp
            const __half2* kh2 = reinterpret_cast<const __half2*>(&kv[u]);
            float dot = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(kh2[e]);
                dot = fmaf(qf[2 * e], f.x, dot);
                dot = fmaf(qf[2 * e + 1], f.y, dot);
            }
#pragma unroll
            for (int msk = 8; msk > 0; msk >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, msk);
            if (k < p1) {
                const float s = dot * scale;
                const float mn = fmaxf(m, s);
                const float corr = (m == -INFINITY) ? 0.0f : expf(m - mn);
                const float pr = expf(s - mn);
                l = l * corr + pr;
                const __half2* vh2 = reinterpret_cast<const __half2*>(&vv[u]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(vh2[e]);
                    o[2 * e] = fmaf(pr, f.x, o[2 * e] * corr);
                    o[2 * e + 1] = fmaf(pr, f.y, o[2 * e + 1] * corr);
                }
                m = mn;
            }
        }
    }
    // CTA-level merge of the 8 half-warp states
#pragma unroll
    for (int e = 0; e < 8; ++e) st[grp * WS_ATT_STRIDE + sl * 8 + e] = o[e];
    if (sl == 0) {
        st[grp * WS_ATT_STRIDE + 128] = m;
        st[grp * WS_ATT_STRIDE + 129] = l;
    }
    __syncthreads();
    float M, L, O;
    att_merge(st, ATT_GROUPS, WS_ATT_STRIDE, tid, M, L, O);
    if (S == 1) {
        ctx[head * 128 + tid] = __float2half_rn(O / L);
        return;
    }
    float* mine = att_part + ((size_t)head * WS_ATT_MAX_SPLITS + split) * WS_ATT_STRIDE;
    mine[tid] = O;
    if (tid == 0) {
        mine[128] = M;
        mine[129] = L;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(&att_count[head], 1);
        s_last = (old == S - 1);
        if (s_last) att_count[head] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* all = att_part + (size_t)head * WS_ATT_MAX_SPLITS * WS_ATT_STRIDE;
    for (int t = tid; t < S * WS_ATT_STRIDE; t += ATT_THREADS) mrg[t] = __ldcg(all + t);
    __syncthreads();
    att_merge(mrg, S, WS_ATT_STRIDE, tid, M, L, O);
    ctx[head * 128 + tid] = __float2half_rn(O / L);
    (void)lane;
}

// ---- host arg-max loop (Inference.cu:1282-1289) on the device --------------------------------------
__device__ __forceinline__ bool better2(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(256)
argmax_kernel(const __half* __restrict__ logits, int n, int* __restrict__ d_token, float* arg_val, int* arg_idx, int* tiles_done) {
    __shared__ float sv[8];
    __shared__ int si[8];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * 1024 + tid; i < min(n, (blockIdx.x + 1) * 1024); i += 256) {
        const float v = __half2float(logits[i]);
        if (better2(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (better2(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp != 0) return;
    bv = lane < 8 ? sv[lane] : -INFINITY;
    bi = lane < 8 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int m = 4; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (better2(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    int last = 0;
    if (lane == 0) {
        arg_val[blockIdx.x] = bv;
        arg_idx[blockIdx.x] = bi;
        __threadfence();
        const int old = atomicAdd(tiles_done, 1);
        last = (old == (int)gridDim.x - 1);
        if (last) *tiles_done = 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (int t = lane; t < (int)gridDim.x; t += 32) {
        const float ov = __ldcg(arg_val + t);
        const int oi = __ldcg(arg_idx + t);
        if (better2(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (better2(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) *d_token = bi;
}

// ---- shared by the C entry points and the engine ---------------------------------------------------
int attn_decode_launch(const void* q, const void* kc, const void* vc, int heads, int head_dim, long long max_pos,
                       const int* d_pos, int pos, void* ctx, const Workspace* ws, bool pdl, cudaStream_t st) {
    QW3_REQUIRE(q && kc && vc && ctx && ws, "qw3_attn_decode: null pointer");
    QW3_REQUIRE(head_dim == 128, "qw3_attn_decode: head_dim must be 128");
    QW3_REQUIRE(heads > 0 && heads <= WS_ATT_MAX_HEADS, "qw3_attn_decode: heads out of range");
    QW3_REQUIRE(d_pos || (pos >= 0 && pos < max_pos), "qw3_attn_decode: pos out of range");
    int S = (2 * ws->sm_count + heads - 1) / heads;
    if (S < 1) S = 1;
    if (S > WS_ATT_MAX_SPLITS) S = WS_ATT_MAX_SPLITS;
    QW3_CUDA(launch(attn_decode_kernel, dim3(heads, S), dim3(ATT_THREADS), 0, st, pdl, static_cast<const __half*>(q),
                    static_cast<const __half*>(kc), static_cast<const __half*>(vc), max_pos, d_pos, pos,
                    static_cast<__half*>(ctx), ws->att_part, ws->att_count));
    return QW3_OK;
}

int embed_gather_launch(const void* packed, const void* scale, const void* zp, long long n_alloc, long long hidden,
                        long long vocab, const int* d_token, const int* d_index, const int* d_skip, int token, void* out,
                        bool pdl, cudaStream_t st) {
    QW3_REQUIRE(packed && scale && zp && out, "qw3_embed_gather_w4: null pointer");
    QW3_REQUIRE(hidden > 0 && vocab > 0 && n_alloc > 0, "qw3_embed_gather_w4: bad shape");
    QW3_REQUIRE(d_token || (token >= 0 && token < vocab), "qw3_embed_gather_w4: token out of range");
    QW3_CUDA(launch(embed_gather_kernel, dim3((unsigned)((hidden + 255) / 256)), dim3(256), 0, st, pdl,
                    static_cast<const uint8_t*>(packed), static_cast<const __half*>(scale), static_cast<const __half*>(zp),
                    n_alloc, (int)hidden, vocab, d_token, d_index, d_skip, token, static_cast<__half*>(out)));
    return QW3_OK;
}

int step_tail_launch(int* d_pos, int* d_step, const int* d_token, int* d_out_ids, int* d_skip, int* d_epoch, bool pdl,
                     cudaStream_t st) {
    QW3_CUDA(launch(step_tail_kernel, dim3(1), dim3(32), 0, st, pdl, d_pos, d_step, d_token, d_out_ids, d_skip, d_epoch));
    return QW3_OK;
}

}  // namespace qw3

using namespace qw3;

extern "C" {

int qw3_dequant_w4(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_alloc, int64_t rows,
                   int64_t cols, void* d_out, void* stream) {
    QW3_REQUIRE(d_packed && d_scale && d_zp && d_out, "qw3_dequant_w4: null pointer");
    QW3_REQUIRE(rows > 0 && cols > 0 && n_alloc > 0, "qw3_dequant_w4: bad shape");
    const long long total = rows * ((cols + 1) / 2);
    const long long blocks = (total + 255) / 256;
    QW3_REQUIRE(blocks <= 0x7fffffffLL, "qw3_dequant_w4: too many elements");
    dequant_w4_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(d_packed), static_cast<const __half*>(d_scale), static_cast<const __half*>(d_zp),
        n_alloc, rows, cols, static_cast<__half*>(d_out));
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

int qw3_rmsnorm(const void* d_x, const void* d_gamma, int64_t n, float eps, void* d_out, void* stream) {
    QW3_REQUIRE(d_x && d_gamma && d_out && n > 0 && n <= 0x7fffffff, "qw3_rmsnorm: bad argument");
    rmsnorm_kernel<<<1, 512, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(d_x),
                                                                      static_cast<const __half*>(d_gamma), (int)n, eps,
                                                                      static_cast<__half*>(d_out));
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

int qw3_rope_kv_append(const void* d_qkv, void* d_q_out, void* d_k_cache, void* d_v_cache, const void* d_cos,
                       const void* d_sin, int32_t heads, int32_t head_dim, int64_t max_pos, const int32_t* d_pos,
                       int32_t pos, void* stream) {
    QW3_REQUIRE(d_qkv && d_q_out && d_k_cache && d_v_cache && d_cos && d_sin, "qw3_rope_kv_append: null pointer");
    QW3_REQUIRE(head_dim == 128 && heads > 0, "qw3_rope_kv_append: head_dim must be 128");
    QW3_REQUIRE(d_pos || (pos >= 0 && pos < max_pos), "qw3_rope_kv_append: pos out of range");
    const int hidden = heads * 128, pairs = 3 * hidden / 2;
    rope_kv_kernel<<<(pairs + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(d_qkv), static_cast<__half*>(d_q_out), static_cast<__half*>(d_k_cache),
        static_cast<__half*>(d_v_cache), static_cast<const __half*>(d_cos), static_cast<const __half*>(d_sin), hidden,
        max_pos, d_pos, pos);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

int qw3_attn_decode(const void* d_q, const void* d_k_cache, const void* d_v_cache, int32_t heads, int32_t head_dim,
                    int64_t max_pos, const int32_t* d_pos, int32_t pos, void* d_ctx, qw3_ws_t ws, void* stream) {
    QW3_REQUIRE(ws, "qw3_attn_decode: null workspace");
    return attn_decode_launch(d_q, d_k_cache, d_v_cache, heads, head_dim, max_pos, d_pos, pos, d_ctx, ws_struct(ws),
                              ws_pdl(ws), static_cast<cudaStream_t>(stream));
}

int qw3_embed_gather_w4(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_alloc, int64_t hidden,
                        int64_t vocab, const int32_t* d_token, int32_t token, void* d_out, void* stream) {
    return embed_gather_launch(d_packed, d_scale, d_zp, n_alloc, hidden, vocab, d_token, nullptr, nullptr, token, d_out, false,
                               static_cast<cudaStream_t>(stream));
}

int qw3_argmax_f16(const void* d_logits, int64_t n, int32_t* d_token, qw3_ws_t ws, void* stream) {
    QW3_REQUIRE(d_logits && d_token && ws, "qw3_argmax_f16: null pointer");
    QW3_REQUIRE(n > 0 && n <= (int64_t)WS_MAX_TILES * 1024, "qw3_argmax_f16: n out of range");
    const Workspace* w = ws_struct(ws);
    argmax_kernel<<<(unsigned)((n + 1023) / 1024), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(d_logits), (int)n, d_token, w->arg_val, w->arg_idx, w->tiles_done);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

}  // extern "C"
