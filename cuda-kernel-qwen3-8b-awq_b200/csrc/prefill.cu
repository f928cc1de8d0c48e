// Batched-row operators of the prompt phase on sm_100a.  The reference runs the prompt one token at a
// time through runOneLayer (Inference.cu:1304-1343); here a block of R prompt tokens goes through a layer
// together: the four projections are the tensor-core W4A16 contraction (gemm_w4a16_tc.cu), and the kernels
// in this file do for R rows what the decode path does for one: embedding gather, RMSNorm, RoPE + KV
// append, causal attention, residual add and GeLU.  The per-element arithmetic (roundings included) is the
// decode path's; only the fp32 summation order inside the contractions differs.
#include "common.cuh"

namespace qw3 {

// ---- gather lambda (Inference.cu:1310-1315) for R tokens: out[r][idx] --------------------------------
__global__ void embed_rows_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scale,
                                  const __half* __restrict__ zp, long long n_alloc, int hidden, long long vocab,
                                  const int* __restrict__ d_tokens, __half* __restrict__ out) {
    const int r = blockIdx.y;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= hidden) return;
    long long tok = d_tokens[r];
    if (tok < 0 || tok >= vocab) tok = 0;   // ids are validated on the host
    const long long pc = (vocab + 1) / 2;
    const uint32_t byte = packed[(long long)idx * pc + (tok >> 1)];
    const uint32_t q = (tok & 1) ? (byte >> 4) : (byte & 15u);
    const long long g = (tok / 128) % n_alloc;
    out[(size_t)r * hidden + idx] = dequant_one(q, zp[g], scale[g]);
}

// ---- rmsNormKernel (Inference.cu:111-145), one CTA per row -----------------------------------------
__global__ void __launch_bounds__(512) rmsnorm_rows_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma,
                                                           int n, float eps, __half* __restrict__ out) {
    __shared__ double dsum[16];
    const __half* xr = x + (size_t)blockIdx.x * n;
    __half* outr = out + (size_t)blockIdx.x * n;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double s = 0.0;
    for (int j = tid; j < n; j += 512) {
        const float v = __half2float(xr[j]);
        s += (double)(v * v);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) s += shfl_xor_double(s, m);
    if (lane == 0) dsum[warp] = s;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int w = 0; w < 16; ++w) tot += dsum[w];
    const float mean_sq = __fdiv_rn((float)tot, (float)n);                                    // Inference.cu:136
    const __half sc = __float2half_rn(__fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps))));  // Inference.cu:137-138
    for (int j = tid; j < n; j += 512) outr[j] = h_mul(h_mul(xr[j], sc), gamma[j]);           // Inference.cu:142-143
}

// ---- QKV split + applyRotaryKernel + KV append (Inference.cu:1070-1103, 150-177) for R rows ---------
// qkv is [R][3*hidden]; q is rotated in place, k (rotated) and v go to cache rows pos0 + r.
__global__ void rope_kv_rows_kernel(__half* __restrict__ qkv, __half* __restrict__ kc, __half* __restrict__ vc,
                                    const __half* __restrict__ cos_t, const __half* __restrict__ sin_t, int hidden,
                                    long long max_pos, int pos0) {
    const int r = blockIdx.y, pos = pos0 + r;
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= 3 * hidden / 2) return;
    const int i = 2 * pair, sec = i / hidden, idx = i - sec * hidden, head = idx >> 7, d = idx & 127;
    __half* row = qkv + (size_t)r * 3 * hidden;
    const __half2 v = *reinterpret_cast<const __half2*>(row + i);
    __half o0 = __low2half(v), o1 = __high2half(v);
    if (sec < 2) {
        const __half cs = cos_t[(size_t)pos * 64 + (d >> 1)], sn = sin_t[(size_t)pos * 64 + (d >> 1)];
        const __half x0 = o0, x1 = o1;
        rope_pair(x0, x1, cs, sn, o0, o1);
    }
    __half* dst = sec == 0 ? row + idx : (sec == 1 ? kc : vc) + ((size_t)head * max_pos + pos) * 128 + d;
    *reinterpret_cast<__half2*>(dst) = __halves2half2(o0, o1);
}

// ---- attentionKernel (Inference.cu:182-266), intended math, causal over a block of R query rows -----
// grid (heads, R), 128 threads: row r attends cache rows 0 .. pos0 + r.  A half-warp owns one cache row at a
// time and keeps an online-softmax state; the 8 states of the CTA are merged in a fixed order.
constexpr int PF_THREADS = 128;
constexpr int PF_GROUPS = PF_THREADS / 16;
constexpr int PF_STRIDE = 132;

__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const __half* __restrict__ qkv, const __half* __restrict__ kc, const __half* __restrict__ vc, int hidden,
                    long long max_pos, int pos0, __half* __restrict__ ctx) {
    __shared__ float st[PF_GROUPS * PF_STRIDE];
    const int head = blockIdx.x, r = blockIdx.y;
    const int tid = threadIdx.x, grp = tid >> 4, sl = tid & 15;
    const int len = pos0 + r + 1;
    float qf[8];
    {
        const uint4 qv = *reinterpret_cast<const uint4*>(qkv + (size_t)r * 3 * hidden + head * 128 + sl * 8);
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
    for (int kb = 0; kb < len; kb += PF_GROUPS * UN) {   // trip count uniform across the CTA
        const int k0 = kb + grp;
        uint4 kv[UN], vv[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int k = k0 + u * PF_GROUPS;
            kv[u] = make_uint4(0, 0, 0, 0);
            vv[u] = make_uint4(0, 0, 0, 0);
            if (k < len) {
                kv[u] = *reinterpret_cast<const uint4*>(kh + (size_t)k * 128);
                vv[u] = *reinterpret_cast<const uint4*>(vh + (size_t)k * 128);
            }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int k = k0 + u * PF_GROUPS;   // uniform within the half-warp
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
            if (k < len) {
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
#pragma unroll
    for (int e = 0; e < 8; ++e) st[grp * PF_STRIDE + sl * 8 + e] = o[e];
    if (sl == 0) {
        st[grp * PF_STRIDE + 128] = m;
        st[grp * PF_STRIDE + 129] = l;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int g = 0; g < PF_GROUPS; ++g) M = fmaxf(M, st[g * PF_STRIDE + 128]);
    float L = 0.0f, O = 0.0f;
    for (int g = 0; g < PF_GROUPS; ++g) {
        const float mg = st[g * PF_STRIDE + 128];
        const float w = (mg == -INFINITY) ? 0.0f : expf(mg - M);
        L += st[g * PF_STRIDE + 129] * w;
        O += st[g * PF_STRIDE + tid] * w;
    }
    ctx[(size_t)r * hidden + head * 128 + tid] = __float2half_rn(O / L);
}

// The residual add (Inference.cu:1145-1156) and the GeLU (Inference.cu:271-279) of the block run in the epilogue of the
// tensor-core contraction that produces their operand.

// ---- launchers used by the engine (all dimensions even; hidden a multiple of 128) --------------------
int embed_rows_launch(const void* packed, const void* scale, const void* zp, long long n_alloc, int hidden, long long vocab,
                      const int* d_tokens, int rows, void* out, cudaStream_t st) {
    embed_rows_kernel<<<dim3((hidden + 255) / 256, rows), 256, 0, st>>>(
        static_cast<const uint8_t*>(packed), static_cast<const __half*>(scale), static_cast<const __half*>(zp), n_alloc, hidden,
        vocab, d_tokens, static_cast<__half*>(out));
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int rmsnorm_rows_launch(const void* x, const void* gamma, int n, float eps, int rows, void* out, cudaStream_t st) {
    rmsnorm_rows_kernel<<<rows, 512, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(gamma), n, eps,
                                              static_cast<__half*>(out));
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int rope_kv_rows_launch(void* qkv, void* kc, void* vc, const void* cos_t, const void* sin_t, int hidden, long long max_pos,
                        int pos0, int rows, cudaStream_t st) {
    rope_kv_rows_kernel<<<dim3((3 * hidden / 2 + 255) / 256, rows), 256, 0, st>>>(
        static_cast<__half*>(qkv), static_cast<__half*>(kc), static_cast<__half*>(vc), static_cast<const __half*>(cos_t),
        static_cast<const __half*>(sin_t), hidden, max_pos, pos0);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int attn_prefill_launch(const void* qkv, const void* kc, const void* vc, int heads, int hidden, long long max_pos, int pos0,
                        int rows, void* ctx, cudaStream_t st) {
    attn_prefill_kernel<<<dim3(heads, rows), PF_THREADS, 0, st>>>(static_cast<const __half*>(qkv), static_cast<const __half*>(kc),
                                                                  static_cast<const __half*>(vc), hidden, max_pos, pos0,
                                                                  static_cast<__half*>(ctx));
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

}  // namespace qw3
