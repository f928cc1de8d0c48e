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

// ---- the same attention on the tensor cores, tiled: 64 query rows x 32 cache rows at a time ------------------------------
// grid (heads, ceil(R / 64)), 4 warps; warp w owns query rows 16w .. 16w+15 of the CTA's block.  A tile of 32 cache rows
// of K and V (8 KB each) is shared by the 64 query rows instead of being read once per row from L2, which is what
// made the row-per-CTA kernel take 1.8 of the 2.0 s of an 8 K prompt.  Per tile and warp: S = Q K^T by 32
// mma.sync.m16n8k16 (fp16 operands, exact products, fp32 sums), online softmax in registers in the accumulator layout,
// O += P V by 32 more (twice) with P as the A operand.  P goes in as TWO fp16 terms (P = hi + lo, lo the rounding error of hi),
// so the probabilities keep 22 bits as in the fp32 arithmetic of the row kernel; V comes in through
// ldmatrix.trans.  K / V tiles are double-buffered with cp.async; rows past the causal limit are zero-filled and masked.
// (mma.sync, not tcgen05: an accumulator that the softmax rescales every tile has to live in registers.)
constexpr int TA_ROWS = 64, TA_KEYS = 32, TA_THREADS = 128, TA_NJ = TA_KEYS / 8;   // (64-key tiles: 8 % slower at 8 K rows, 16-key tiles 20 %)
constexpr int TA_LD = 136;                                   // halves per shared-memory row (272 B: ldmatrix rows 16-byte aligned, no bank conflicts)
constexpr size_t TA_TILE = (size_t)TA_KEYS * TA_LD * 2;      // bytes of one K or V tile
constexpr size_t TA_SMEM = (size_t)TA_ROWS * TA_LD * 2 + 4 * TA_TILE;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_h(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared; `valid` false: the 16 bytes are zero-filled (the source is not read)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void split_hi_lo(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

__global__ void __launch_bounds__(TA_THREADS, 4)   // 52 KB of shared memory and 128 registers: four CTAs per SM
attn_prefill_tiled_kernel(const __half* __restrict__ qkv, const __half* __restrict__ kc, const __half* __restrict__ vc, int hidden,
                          long long max_pos, int pos0, int rows, __half* __restrict__ ctx) {
    extern __shared__ __align__(128) uint8_t ta_smem[];
    const int head = blockIdx.x, r0 = (gridDim.y - 1 - blockIdx.y) * TA_ROWS;   // the row blocks with the most cache rows start first
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t q_s = smem_u32(ta_smem), kv_s = q_s + TA_ROWS * TA_LD * 2;   // kv_s + (2 * stage + {0: K, 1: V}) * TA_TILE
    const int n_rows = min(TA_ROWS, rows - r0);
    const int n_keys = pos0 + r0 + n_rows;                       // cache rows any query row of this block may see
    const int n_tiles = (n_keys + TA_KEYS - 1) / TA_KEYS;
    const __half* kh = kc + (size_t)head * max_pos * 128;
    const __half* vh = vc + (size_t)head * max_pos * 128;
    auto load_tile = [&](int tile, int stage) {
        const int k0 = tile * TA_KEYS;
        for (int i = tid; i < TA_KEYS * 16; i += TA_THREADS) {   // 16-byte pieces: 16 per cache row
            const int row = i >> 4, piece = i & 15, key = k0 + row;
            const bool ok = key < n_keys;
            const size_t src = (size_t)(ok ? key : 0) * 128 + piece * 8;
            const uint32_t dst = (uint32_t)(row * TA_LD + piece * 8) * 2;
            cp_async16(kv_s + (2 * stage) * TA_TILE + dst, kh + src, ok);
            cp_async16(kv_s + (2 * stage + 1) * TA_TILE + dst, vh + src, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(0, 0);
    for (int i = tid; i < TA_ROWS * 16; i += TA_THREADS) {       // the block's q rows (after RoPE), zero past the last row
        const int row = i >> 4, piece = i & 15;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows) v = *reinterpret_cast<const uint4*>(qkv + (size_t)(r0 + row) * 3 * hidden + head * 128 + piece * 8);
        *reinterpret_cast<uint4*>(ta_smem + (size_t)(row * TA_LD + piece * 8) * 2) = v;
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int d = 0; d < 4; ++d) o[n][d] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;   // rows g and g + 8 of the warp's 16
    const float scale = 1.0f / sqrtf(128.0f);                             // Inference.cu:218
    const int pos_lo = pos0 + r0 + warp * 16 + g, pos_hi = pos_lo + 8;    // last cache row each of the two query rows sees
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) {
            load_tile(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // the tile (and, the first time, the q rows) are in shared memory
        const uint32_t k_s = kv_s + (2 * stage) * TA_TILE, v_s = k_s + TA_TILE;
        // ---- S = Q K^T: 16 rows x 64 keys per warp
        float sc[TA_NJ][4];
#pragma unroll
        for (int j = 0; j < TA_NJ; ++j)
#pragma unroll
            for (int d = 0; d < 4; ++d) sc[j][d] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(q_s + (uint32_t)((warp * 16 + (lane & 15)) * TA_LD + kk * 16 + 8 * (lane >> 4)) * 2, a0, a1, a2, a3);
#pragma unroll
            for (int j = 0; j < TA_NJ; j += 2) {   // two key tiles per ldmatrix: (b0, b1) of tile j, then of tile j + 1
                uint32_t b0, b1, b2, b3;
                ldsm_x4(k_s + (uint32_t)((j * 8 + (lane & 7) + 8 * (lane >> 4)) * TA_LD + kk * 16 + 8 * ((lane >> 3) & 1)) * 2, b0, b1, b2, b3);
                mma_h(sc[j], a0, a1, a2, a3, b0, b1);
                mma_h(sc[j + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- scale, causal mask, online softmax (rows g: regs 0, 1; rows g + 8: regs 2, 3; keys 8j + 2t, + 1)
        const int k0 = tile * TA_KEYS;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < TA_NJ; ++j) {
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const int key = k0 + j * 8 + 2 * t + (d & 1);
                const bool ok = key <= ((d & 2) ? pos_hi : pos_lo);
                sc[j][d] = ok ? sc[j][d] * scale : -INFINITY;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(sc[j][0], sc[j][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(sc[j][2], sc[j][3]));
        }
#pragma unroll
        for (int msk = 1; msk <= 2; msk <<= 1) {
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, msk));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, msk));
        }
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float c_lo = (m_lo == -INFINITY) ? 0.0f : expf(m_lo - mn_lo), c_hi = (m_hi == -INFINITY) ? 0.0f : expf(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        l_lo *= c_lo;
        l_hi *= c_hi;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            o[n][0] *= c_lo; o[n][1] *= c_lo;
            o[n][2] *= c_hi; o[n][3] *= c_hi;
        }
#pragma unroll
        for (int j = 0; j < TA_NJ; ++j) {   // a row with nothing visible yet (only rows past the block's end) keeps p = 0
            sc[j][0] = (mn_lo == -INFINITY) ? 0.0f : expf(sc[j][0] - mn_lo);
            sc[j][1] = (mn_lo == -INFINITY) ? 0.0f : expf(sc[j][1] - mn_lo);
            sc[j][2] = (mn_hi == -INFINITY) ? 0.0f : expf(sc[j][2] - mn_hi);
            sc[j][3] = (mn_hi == -INFINITY) ? 0.0f : expf(sc[j][3] - mn_hi);
            l_lo += sc[j][0] + sc[j][1];
            l_hi += sc[j][2] + sc[j][3];
        }
        // ---- O += P V: P (16 x 64) as A operand, hi and lo terms; V through ldmatrix.trans
#pragma unroll
        for (int kk = 0; kk < TA_KEYS / 16; ++kk) {   // 16 keys: score tiles 2kk and 2kk + 1
            uint32_t h0, h1, h2, h3, e0, e1, e2, e3;
            split_hi_lo(sc[2 * kk][0], sc[2 * kk][1], h0, e0);
            split_hi_lo(sc[2 * kk][2], sc[2 * kk][3], h1, e1);
            split_hi_lo(sc[2 * kk + 1][0], sc[2 * kk + 1][1], h2, e2);
            split_hi_lo(sc[2 * kk + 1][2], sc[2 * kk + 1][3], h3, e3);
#pragma unroll
            for (int n = 0; n < 16; n += 2) {   // two tiles of 8 dims per ldmatrix
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(v_s + (uint32_t)((kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * TA_LD + n * 8 + 8 * (lane >> 4)) * 2, b0, b1, b2, b3);
                mma_h(o[n], h0, h1, h2, h3, b0, b1);
                mma_h(o[n], e0, e1, e2, e3, b0, b1);
                mma_h(o[n + 1], h0, h1, h2, h3, b2, b3);
                mma_h(o[n + 1], e0, e1, e2, e3, b2, b3);
            }
        }
        __syncthreads();   // everybody is done with this stage before the tile after next lands in it
    }
#pragma unroll
    for (int msk = 1; msk <= 2; msk <<= 1) {
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, msk);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, msk);
    }
    const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        if (row_lo < n_rows)
            *reinterpret_cast<__half2*>(ctx + (size_t)(r0 + row_lo) * hidden + head * 128 + n * 8 + 2 * t) =
                __floats2half2_rn(o[n][0] / l_lo, o[n][1] / l_lo);   // one rounding to fp16, Inference.cu:257-265
        if (row_hi < n_rows)
            *reinterpret_cast<__half2*>(ctx + (size_t)(r0 + row_hi) * hidden + head * 128 + n * 8 + 2 * t) =
                __floats2half2_rn(o[n][2] / l_hi, o[n][3] / l_hi);
    }
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
    if (rows >= 16) {   // blocks of rows: the tiled tensor-core kernel; a few rows: one CTA per row
        static bool attr_set[64] = {};   // per device: the kernel's shared-memory limit is raised once
        int dev = 0;
        QW3_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) {
            QW3_CUDA(cudaFuncSetAttribute(attn_prefill_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TA_SMEM));
        } else if (!attr_set[dev]) {
            QW3_CUDA(cudaFuncSetAttribute(attn_prefill_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TA_SMEM));
            attr_set[dev] = true;
        }
        attn_prefill_tiled_kernel<<<dim3(heads, (rows + TA_ROWS - 1) / TA_ROWS), TA_THREADS, TA_SMEM, st>>>(
            static_cast<const __half*>(qkv), static_cast<const __half*>(kc), static_cast<const __half*>(vc), hidden, max_pos, pos0,
            rows, static_cast<__half*>(ctx));
    } else {
        attn_prefill_kernel<<<dim3(heads, rows), PF_THREADS, 0, st>>>(static_cast<const __half*>(qkv), static_cast<const __half*>(kc),
                                                                      static_cast<const __half*>(vc), hidden, max_pos, pos0,
                                                                      static_cast<__half*>(ctx));
    }
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

}  // namespace qw3

extern "C" int qw3_attn_prefill(const void* d_qkv, const void* d_k_cache, const void* d_v_cache, int32_t heads, int32_t head_dim,
                                int64_t max_pos, int32_t pos0, int32_t rows, void* d_ctx, void* stream) {
    QW3_REQUIRE(d_qkv && d_k_cache && d_v_cache && d_ctx, "qw3_attn_prefill: null pointer");
    QW3_REQUIRE(head_dim == 128 && heads > 0, "qw3_attn_prefill: head_dim must be 128, heads positive");
    QW3_REQUIRE(rows > 0 && pos0 >= 0 && (int64_t)pos0 + rows <= max_pos, "qw3_attn_prefill: rows out of range");
    return qw3::attn_prefill_launch(d_qkv, d_k_cache, d_v_cache, heads, heads * 128, max_pos, pos0, rows, d_ctx,
                                    static_cast<cudaStream_t>(stream));
}
