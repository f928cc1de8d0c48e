// Fused AWQ dequantise + matrix-vector product for one token (batch-1 decode) on sm_100a.
//
// Replaces, per call, dequantAwqKernel (Inference.cu:76-106, run once at load in the reference)
// plus one cublasGemmEx at n = 1 (Inference.cu:1052, 1128, 1176, 1201, 1260) and the small kernel
// that follows it (RoPE + KV append, residual add, GeLU, fp16->fp32 + host arg-max).
//
// Data layout.  The packed file is a flat nibble stream; the reference's GEMM reads its fp16
// expansion column-major with lda = out_dim, so input j owns out_dim consecutive nibbles:
// bytes [K][M/2], and y[i] = sum_j w(i, j) x[j] reduces ACROSS rows.  Scale / zero-point of
// element (i, j): g = ((i/128 + j*(M/128)) mod (K/128)) mod n_alloc.
//
// Kernel.  One persistent CTA per SM.  The (tile, row) space -- tiles of 1024 outputs (512 B of
// every row), units of 8 rows (one 4 KB TMA box) -- is flattened and cut into equal contiguous
// ranges, one per CTA, so every SM streams the same number of bytes whatever the shape.  A
// producer lane keeps a 4 x 32 KB ring of TMA boxes in flight; 16 consumer warps each take 4
// rows x 1024 outputs of a stage: a lane owns 32 consecutive outputs, unpacks nibble pairs with
// one lop3 each into (1024+q) halves, applies the reference's two roundings (q - zp, * scale) in
// packed fp16, and accumulates in fp32 on the tensor cores: the two halves of a register are two
// outputs of one input row, separated by the column of B that holds x[row]
// (B[k][n] = x if k = n mod 8), so D needs no cross-lane exchange.  Partial sums of a tile that
// spans CTAs go to scratch; the last CTA to arrive adds them in CTA order (deterministic) and
// runs the epilogue.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace qw3 {

constexpr int TI = WS_TILE;                       // outputs per tile
constexpr int ROW_BYTES = TI / 2;                 // 512
constexpr int UNIT_ROWS = 8;
constexpr int UNIT_BYTES = UNIT_ROWS * ROW_BYTES; // 4096: one TMA box
constexpr int NCW = 16;                           // consumer warps
constexpr int STAGE_UNITS = 8;                    // 64 rows
constexpr int STAGE_BYTES = STAGE_UNITS * UNIT_BYTES;
constexpr int NSTAGES = 4;
constexpr int NCONS = NCW * 32;
constexpr int NTHREADS = NCONS + 32;
constexpr int MAX_GROUPS = 256;
constexpr int RED_BYTES = 4 * TI * 4;
constexpr int MISC_BYTES = 512;

struct GemvParams {
    const __half* scale;
    const __half* zp;
    int n_alloc;
    int M, K, Mb, Kb;
    int n_tiles, upt;   // tiles of TI outputs; units (8 rows) per tile
    long long U;        // n_tiles * upt
    const __half* x;
    const __half* gamma;
    float eps;
    int epilogue;
    __half* y;
    __half* kc;
    __half* vc;
    const __half* cos_t;
    const __half* sin_t;
    int hidden;         // M / 3 for ROPE_KV
    long long max_pos;
    const int* d_pos;
    int pos;
    int* d_token;
    float* logits_f32;
    Workspace ws;
};

template <bool UNIFORM, bool EXACT>
__global__ void __launch_bounds__(NTHREADS, 1)
gemv_w4a16_kernel(const __grid_constant__ CUtensorMap tmap, const GemvParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + NSTAGES * STAGE_BYTES);
    __half* xs = reinterpret_cast<__half*>(smem + NSTAGES * STAGE_BYTES + RED_BYTES);
    uint8_t* after_x = smem + NSTAGES * STAGE_BYTES + RED_BYTES + (size_t)p.K * 2;
    uint16_t* gidx = reinterpret_cast<uint16_t*>(after_x);                                   // [K]   (non-uniform)
    uint4* gtab = reinterpret_cast<uint4*>(after_x + (UNIFORM ? 0 : (size_t)p.K * 2));       // [256] (non-uniform)
    uint8_t* misc = reinterpret_cast<uint8_t*>(gtab) + (UNIFORM ? 0 : MAX_GROUPS * 16);
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc);             // full[4], empty[4]
    double* dsum = reinterpret_cast<double*>(misc + 64);            // [16]
    float* s_argv = reinterpret_cast<float*>(misc + 192);           // [16]
    int* s_argi = reinterpret_cast<int*>(misc + 256);               // [16]
    int* s_flag = reinterpret_cast<int*>(misc + 320);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + NSTAGES);

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, NCW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const int G = gridDim.x, c = blockIdx.x;
    const long long U = p.U;
    const long long u_begin = (long long)c * U / G, u_end = (long long)(c + 1) * U / G;
    const int upt = p.upt;

    if (warp == NCW) {
        // ---------------- producer: weights do not depend on the previous kernel, start at once.
        if (lane == 0) {
            tma_prefetch_desc(&tmap);
            int it = 0;
            for (long long u = u_begin; u < u_end; ++it) {
                const int tile = (int)(u / upt), r = (int)(u - (long long)tile * upt);
                long long n64 = u_end - u;
                int n = upt - r < STAGE_UNITS ? upt - r : STAGE_UNITS;
                if (n64 < n) n = (int)n64;
                const int slot = it % NSTAGES;
                const uint32_t ph = (it / NSTAGES) & 1;
                if (it >= NSTAGES && !mbar_wait(empty0 + 8 * slot, ph ^ 1)) {
                    atomicExch(p.ws.err, QW3_ERR_TIMEOUT);
                    break;
                }
                mbar_expect_tx(full0 + 8 * slot, (uint32_t)n * UNIT_BYTES);
                const uint32_t dst = smem_u32(ring + slot * STAGE_BYTES);
                for (int k = 0; k < n; ++k)
                    tma_load_2d(dst + k * UNIT_BYTES, &tmap, tile * (TI / 8), (r + k) * UNIT_ROWS, full0 + 8 * slot);
                u += n;
            }
        }
        return;
    }

    // ---------------- consumers ------------------------------------------------------------------
    pdl_wait();  // x, gamma-normalised input, residual and scratch belong to earlier kernels

    // Prologue: (optionally RMS-normalised) x -> shared; group tables for j-dependent groups.
    __half nscale = __ushort_as_half(0x3C00);
    if (p.gamma != nullptr) {
        double s = 0.0;
        for (int j = tid; j < p.K; j += NCONS) {
            const float v = __half2float(p.x[j]);
            s += (double)(v * v);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) s += shfl_xor_double(s, m);
        if (lane == 0) dsum[warp] = s;
        named_barrier(1, NCONS);
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < NCW; ++w) tot += dsum[w];
        const float mean_sq = __fdiv_rn((float)tot, (float)p.K);                       // Inference.cu:136
        const float denom = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, p.eps)));    // Inference.cu:137
        nscale = __float2half_rn(denom);                                               // Inference.cu:138
        for (int j = tid; j < p.K; j += NCONS) xs[j] = h_mul(h_mul(p.x[j], nscale), p.gamma[j]);  // :142-143
    } else {
        for (int j = tid; j < p.K; j += NCONS) xs[j] = p.x[j];
    }
    if (!UNIFORM) {
        for (int j = tid; j < p.K; j += NCONS) gidx[j] = (uint16_t)(((long long)j * p.Mb) % p.Kb);
        const int n_used = p.Kb < p.n_alloc ? p.Kb : p.n_alloc;
        for (int g = tid; g < n_used; g += NCONS) {
            const DqConst k = make_const<EXACT>(p.zp[g], p.scale[g]);
            gtab[g] = make_uint4(k.z, k.hz, k.s, 0u);
        }
    }
    named_barrier(1, NCONS);

    float acc[4][2][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int d = 0; d < 4; ++d) acc[a][b][d] = 0.0f;

    // Lane (q, t) holds column n = q of B: non-zero only where k = q (mod 8), i.e. t == q/2,
    // in the half selected by q & 1.
    const int q4 = lane >> 2, t4 = lane & 3;
    const bool is_b = (t4 == (q4 >> 1));
    const int bshift = (q4 & 1) * 16;

    bool dead = false;
    int cur_tile = -1;
    DqConst ku = {0u, 0u, 0u};
    int ibk = 0;

    auto flush = [&](int tile) {
        // 1. cross-warp reduction in a fixed order: red[s] = ((w_s + w_{s+4}) + w_{s+8}) + w_{s+12}
        float* mine = red + (warp & 3) * TI + lane * 32;
#pragma unroll
        for (int round = 0; round < 4; ++round) {
            if ((warp >> 2) == round) {
#pragma unroll
                for (int wd = 0; wd < 4; ++wd)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int d = 0; d < 4; ++d) {
                            // d0:(lo,low) d1:(lo,high) d2:(hi,low) d3:(hi,high) -> nibble index
                            const int nib = (d >> 1) + ((d & 1) << 2) + (h << 1);
                            const int off = (8 * wd + nib + lane) & 31;  // skewed: conflict-free
                            if (round == 0) mine[off] = acc[wd][h][d];
                            else mine[off] += acc[wd][h][d];
                            acc[wd][h][d] = 0.0f;
                        }
            }
            named_barrier(1, NCONS);
        }
        float tot[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int il = 2 * tid + e, ln = il >> 5, pos = ln * 32 + (((il & 31) + ln) & 31);
            tot[e] = ((red[pos] + red[TI + pos]) + red[2 * TI + pos]) + red[3 * TI + pos];
        }
        named_barrier(1, NCONS);  // red may be rewritten by the next flush

        // 2. cross-CTA fix-up when the tile's rows are shared between CTAs
        const long long ut0 = (long long)tile * upt;
        const int cf = owner_of(ut0, G, U), cl = owner_of(ut0 + upt - 1, G, U);
        if (cf != cl) {
            float* part = p.ws.partials + (size_t)(c + tile) * TI;
            *reinterpret_cast<float2*>(part + 2 * tid) = make_float2(tot[0], tot[1]);
            __threadfence();
            named_barrier(1, NCONS);
            if (tid == 0) {
                const int old = atomicAdd(&p.ws.counters[tile], 1);
                const int last = (old == cl - cf);
                if (last) p.ws.counters[tile] = 0;
                *s_flag = last;
            }
            named_barrier(1, NCONS);
            const int last = *s_flag;
            named_barrier(1, NCONS);  // s_flag may be rewritten by the next flush
            if (!last) return;
            __threadfence();
            tot[0] = 0.0f;
            tot[1] = 0.0f;
            for (int cc = cf; cc <= cl; ++cc) {
                const float2 v = __ldcg(reinterpret_cast<const float2*>(p.ws.partials + (size_t)(cc + tile) * TI + 2 * tid));
                tot[0] += v.x;
                tot[1] += v.y;
            }
        }

        // 3. epilogue on outputs i, i+1
        const int i = tile * TI + 2 * tid;
        const bool valid = i < p.M;
        const __half h0 = __float2half_rn(tot[0]), h1 = __float2half_rn(tot[1]);
        if (p.epilogue == QW3_EPI_STORE) {
            if (valid) *reinterpret_cast<__half2*>(p.y + i) = __halves2half2(h0, h1);
        } else if (p.epilogue == QW3_EPI_RESIDUAL) {
            if (valid) {
                const __half2 r = *reinterpret_cast<const __half2*>(p.y + i);
                *reinterpret_cast<__half2*>(p.y + i) = __halves2half2(h_add(__low2half(r), h0), h_add(__high2half(r), h1));
            }
        } else if (p.epilogue == QW3_EPI_GELU) {
            if (valid) *reinterpret_cast<__half2*>(p.y + i) = __halves2half2(gelu_h(h0), gelu_h(h1));
        } else if (p.epilogue == QW3_EPI_ROPE_KV) {
            if (valid) {
                const int pos = p.d_pos ? *p.d_pos : p.pos;
                const int sec = i / p.hidden, idx = i - sec * p.hidden;   // 0 = Q, 1 = K, 2 = V
                const int head = idx >> 7, d = idx & 127;
                __half o0 = h0, o1 = h1;
                if (sec < 2) {                                            // Inference.cu:166-176
                    const __half cs = p.cos_t[(size_t)pos * 64 + (d >> 1)], sn = p.sin_t[(size_t)pos * 64 + (d >> 1)];
                    rope_pair(h0, h1, cs, sn, o0, o1);
                }
                __half* dst = sec == 0 ? p.y + idx
                                       : (sec == 1 ? p.kc : p.vc) + ((size_t)head * p.max_pos + pos) * 128 + d;
                *reinterpret_cast<__half2*>(dst) = __halves2half2(o0, o1);
            }
        } else {  // QW3_EPI_ARGMAX
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            if (valid) {
                if (p.y) *reinterpret_cast<__half2*>(p.y + i) = __halves2half2(h0, h1);
                const float f0 = __half2float(h0), f1 = __half2float(h1);
                if (p.logits_f32) *reinterpret_cast<float2*>(p.logits_f32 + i) = make_float2(f0, f1);
                bv = f0; bi = i;
                if (f1 > f0) { bv = f1; bi = i + 1; }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { s_argv[warp] = bv; s_argi[warp] = bi; }
            named_barrier(1, NCONS);
            if (warp == 0) {
                bv = lane < NCW ? s_argv[lane] : -INFINITY;
                bi = lane < NCW ? s_argi[lane] : 0x7fffffff;
#pragma unroll
                for (int m = 8; m > 0; m >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                }
                int last = 0;
                if (lane == 0) {
                    p.ws.arg_val[tile] = bv;
                    p.ws.arg_idx[tile] = bi;
                    __threadfence();
                    const int old = atomicAdd(p.ws.tiles_done, 1);
                    last = (old == p.n_tiles - 1);
                    if (last) *p.ws.tiles_done = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {  // whole-vocabulary winner: lowest index among equal maxima
                    __threadfence();
                    bv = -INFINITY; bi = 0x7fffffff;
                    for (int t = lane; t < p.n_tiles; t += 32) {
                        const float ov = __ldcg(p.ws.arg_val + t);
                        const int oi = __ldcg(p.ws.arg_idx + t);
                        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                    }
#pragma unroll
                    for (int m = 16; m > 0; m >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                    }
                    if (lane == 0 && p.d_token) *p.d_token = bi;
                }
            }
            named_barrier(1, NCONS);  // s_argv / s_argi may be rewritten by the next flush
        }
    };

    int it = 0;
    for (long long u = u_begin; u < u_end; ++it) {
        const int tile = (int)(u / upt), r = (int)(u - (long long)tile * upt);
        long long n64 = u_end - u;
        int n = upt - r < STAGE_UNITS ? upt - r : STAGE_UNITS;
        if (n64 < n) n = (int)n64;
        if (tile != cur_tile) {
            if (cur_tile >= 0) flush(cur_tile);
            cur_tile = tile;
            int ib = tile * (TI / 128) + (lane >> 2);
            if (ib >= p.Mb) ib = 0;  // columns past out_dim: zero-filled by TMA, results discarded
            ibk = ib % p.Kb;
            if (UNIFORM) {
                const int g = ibk % p.n_alloc;
                ku = make_const<EXACT>(p.zp[g], p.scale[g]);
            }
        }
        const int slot = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        if (!dead && !mbar_wait(full0 + 8 * slot, ph)) {
            dead = true;  // keep the control flow (barriers, arrivals) uniform; results are void
            if (lane == 0) atomicExch(p.ws.err, QW3_ERR_TIMEOUT);
        }
        const int unit = warp >> 1;
        if (!dead && unit < n) {
            const int jrow = (r + unit) * UNIT_ROWS + (warp & 1) * 4;   // first of this warp's 4 rows
            const uint8_t* src = ring + slot * STAGE_BYTES + unit * UNIT_BYTES + (warp & 1) * 4 * ROW_BYTES + lane * 16;
            const uint4 ra = *reinterpret_cast<const uint4*>(src);
            const uint4 rb = *reinterpret_cast<const uint4*>(src + ROW_BYTES);
            const uint4 rc = *reinterpret_cast<const uint4*>(src + 2 * ROW_BYTES);
            const uint4 rd = *reinterpret_cast<const uint4*>(src + 3 * ROW_BYTES);
            const uint2 xv = *reinterpret_cast<const uint2*>(xs + jrow);
            const uint32_t bac0 = is_b ? ((xv.x & 0xffffu) << bshift) : 0u;   // x[row a]
            const uint32_t bbd0 = is_b ? ((xv.x >> 16) << bshift) : 0u;       // x[row b]
            const uint32_t bac1 = is_b ? ((xv.y & 0xffffu) << bshift) : 0u;   // x[row c]
            const uint32_t bbd1 = is_b ? ((xv.y >> 16) << bshift) : 0u;       // x[row d]
            DqConst ka = ku, kb = ku, kc = ku, kd = ku;
            if (!UNIFORM) {
                const uint2 gv = *reinterpret_cast<const uint2*>(gidx + jrow);
                int g0 = ibk + (int)(gv.x & 0xffffu), g1 = ibk + (int)(gv.x >> 16);
                int g2 = ibk + (int)(gv.y & 0xffffu), g3 = ibk + (int)(gv.y >> 16);
                g0 -= g0 >= p.Kb ? p.Kb : 0; g1 -= g1 >= p.Kb ? p.Kb : 0;
                g2 -= g2 >= p.Kb ? p.Kb : 0; g3 -= g3 >= p.Kb ? p.Kb : 0;
                if (p.Kb > p.n_alloc) { g0 %= p.n_alloc; g1 %= p.n_alloc; g2 %= p.n_alloc; g3 %= p.n_alloc; }
                uint4 t;
                t = gtab[g0]; ka = {t.x, t.y, t.z};
                t = gtab[g1]; kb = {t.x, t.y, t.z};
                t = gtab[g2]; kc = {t.x, t.y, t.z};
                t = gtab[g3]; kd = {t.x, t.y, t.z};
            }
            const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w}, wb[4] = {rb.x, rb.y, rb.z, rb.w};
            const uint32_t wc[4] = {rc.x, rc.y, rc.z, rc.w}, wdd[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t alo, ahi, blo, bhi, clo, chi, dlo, dhi;
                    dq_pair<EXACT>(h ? wa[wd] >> 8 : wa[wd], ka, alo, ahi);
                    dq_pair<EXACT>(h ? wc[wd] >> 8 : wc[wd], kc, clo, chi);
                    mma_16816(acc[wd][h], alo, ahi, clo, chi, bac0, bac1);
                    dq_pair<EXACT>(h ? wb[wd] >> 8 : wb[wd], kb, blo, bhi);
                    dq_pair<EXACT>(h ? wdd[wd] >> 8 : wdd[wd], kd, dlo, dhi);
                    mma_16816(acc[wd][h], blo, bhi, dlo, dhi, bbd0, bbd1);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * slot);
        u += n;
    }
    if (cur_tile >= 0) flush(cur_tile);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------

static thread_local char g_last_error[512] = "";
void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

int encode_2d_u32(CUtensorMap* map, const void* base, uint64_t inner_elems, uint64_t rows, uint64_t pitch_bytes,
                  uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
        return QW3_ERR_CUDA;
    }
    cuuint64_t dims[2] = {inner_elems, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return QW3_ERR_CUDA;
    }
    return QW3_OK;
}

size_t workspace_bytes() {
    size_t b = 0;
    b += (size_t)(WS_MAX_CTAS + WS_MAX_TILES) * WS_TILE * 4;  // partials
    b += (size_t)WS_MAX_TILES * 4;                            // counters
    b += 256;                                                 // tiles_done
    b += (size_t)WS_MAX_TILES * 4 * 2;                        // arg_val, arg_idx
    b += (size_t)WS_ATT_MAX_HEADS * WS_ATT_MAX_SPLITS * WS_ATT_STRIDE * 4;
    b += (size_t)WS_ATT_MAX_HEADS * 4;
    b += 256;                                                 // err
    return b;
}

void workspace_carve(Workspace* ws, void* base) {
    uint8_t* p = static_cast<uint8_t*>(base);
    ws->partials = reinterpret_cast<float*>(p);   p += (size_t)(WS_MAX_CTAS + WS_MAX_TILES) * WS_TILE * 4;
    ws->counters = reinterpret_cast<int32_t*>(p); p += (size_t)WS_MAX_TILES * 4;
    ws->tiles_done = reinterpret_cast<int32_t*>(p); p += 256;
    ws->arg_val = reinterpret_cast<float*>(p);    p += (size_t)WS_MAX_TILES * 4;
    ws->arg_idx = reinterpret_cast<int32_t*>(p);  p += (size_t)WS_MAX_TILES * 4;
    ws->att_part = reinterpret_cast<float*>(p);   p += (size_t)WS_ATT_MAX_HEADS * WS_ATT_MAX_SPLITS * WS_ATT_STRIDE * 4;
    ws->att_count = reinterpret_cast<int32_t*>(p); p += (size_t)WS_ATT_MAX_HEADS * 4;
    ws->err = reinterpret_cast<int32_t*>(p);
}

// Byte offset (within the workspace allocation) from which everything must start at zero.
static size_t workspace_zero_from() { return (size_t)(WS_MAX_CTAS + WS_MAX_TILES) * WS_TILE * 4; }

static size_t gemv_smem_bytes(int K, bool uniform) {
    size_t b = (size_t)NSTAGES * STAGE_BYTES + RED_BYTES + (size_t)K * 2;
    if (!uniform) b += (size_t)K * 2 + MAX_GROUPS * 16;
    return b + MISC_BYTES;
}

template <bool UNIFORM, bool EXACT>
static int launch_gemv(const W4Desc* w, const GemvParams& p, int grid, size_t smem, bool pdl, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    QW3_CUDA(cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<UNIFORM, EXACT>, w->tmap, p));
    return QW3_OK;
}

// Opt every instantiation in to the large dynamic shared-memory carve-out on the current device
// (done when a workspace is created, never inside a stream capture).
static int gemv_init_device() {
    QW3_CUDA(cudaFuncSetAttribute(gemv_w4a16_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    QW3_CUDA(cudaFuncSetAttribute(gemv_w4a16_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    QW3_CUDA(cudaFuncSetAttribute(gemv_w4a16_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    QW3_CUDA(cudaFuncSetAttribute(gemv_w4a16_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return QW3_OK;
}

struct WsHandle {
    Workspace ws;
    int use_pdl;
};

}  // namespace qw3

using namespace qw3;

struct qw3_w4 { W4Desc d; };
struct qw3_ws { WsHandle h; };

extern "C" {

const char* qw3_last_error(void) { return g_last_error; }

const char* qw3_strerror(int s) {
    switch (s) {
        case QW3_OK: return "ok";
        case QW3_ERR_ARG: return "bad argument or unsupported shape";
        case QW3_ERR_CUDA: return "CUDA call failed";
        case QW3_ERR_IO: return "weight file missing or too short";
        case QW3_ERR_RANGE: return "sequence exceeds the KV capacity or token id out of range";
        case QW3_ERR_TIMEOUT: return "bounded device-side wait gave up";
        case QW3_ERR_DEVICE: return "not enough GPUs or peer access unavailable";
        case QW3_ERR_NOMEM: return "out of memory";
        case QW3_ERR_STATE: return "call not valid in this state";
        default: return "unknown status";
    }
}

int qw3_w4_create(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_alloc, int64_t out_dim,
                  int64_t in_dim, int zp_integral, qw3_w4_t* out) {
    QW3_REQUIRE(out && d_packed && d_scale && d_zp, "qw3_w4_create: null pointer");
    QW3_REQUIRE(out_dim > 0 && in_dim > 0 && out_dim % 128 == 0 && in_dim % 128 == 0,
                "qw3_w4_create: out_dim=%lld and in_dim=%lld must be positive multiples of 128", (long long)out_dim, (long long)in_dim);
    QW3_REQUIRE(n_alloc > 0 && n_alloc <= 0x7fffffff, "qw3_w4_create: n_groups_alloc out of range");
    QW3_REQUIRE(out_dim <= (int64_t)WS_MAX_TILES * WS_TILE && in_dim <= 32768, "qw3_w4_create: shape too large");
    QW3_REQUIRE((reinterpret_cast<uintptr_t>(d_packed) & 15) == 0, "qw3_w4_create: packed pointer must be 16-byte aligned");
    qw3_w4* w = new (std::nothrow) qw3_w4();
    if (!w) return QW3_ERR_NOMEM;
    W4Desc& d = w->d;
    d.packed = static_cast<const uint8_t*>(d_packed);
    d.scale = static_cast<const __half*>(d_scale);
    d.zp = static_cast<const __half*>(d_zp);
    d.n_alloc = n_alloc; d.M = out_dim; d.K = in_dim; d.zp_integral = zp_integral ? 1 : 0;
    const int64_t Mb = out_dim / 128, Kb = in_dim / 128;
    d.uniform = (Mb % Kb == 0) || (Kb % n_alloc == 0 && Mb % n_alloc == 0);
    int rc = encode_2d_u32(&d.tmap, d_packed, (uint64_t)out_dim / 8, (uint64_t)in_dim, (uint64_t)out_dim / 2,
                           TI / 8, UNIT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != QW3_OK) { delete w; return rc; }
    *out = w;
    return QW3_OK;
}

int qw3_w4_destroy(qw3_w4_t w) {
    delete w;
    return QW3_OK;
}

int qw3_ws_create(qw3_ws_t* out) {
    QW3_REQUIRE(out, "qw3_ws_create: null pointer");
    {
        const int rc = gemv_init_device();
        if (rc != QW3_OK) return rc;
    }
    qw3_ws* h = new (std::nothrow) qw3_ws();
    if (!h) return QW3_ERR_NOMEM;
    void* base = nullptr;
    cudaError_t e = cudaMalloc(&base, workspace_bytes());
    if (e != cudaSuccess) {
        set_last_error("qw3_ws_create: cudaMalloc(%zu) -> %s", workspace_bytes(), cudaGetErrorString(e));
        delete h;
        return QW3_ERR_CUDA;
    }
    workspace_carve(&h->h.ws, base);
    h->h.ws.base = base;
    h->h.use_pdl = 0;
    cudaGetDevice(&h->h.ws.device);
    cudaDeviceGetAttribute(&h->h.ws.sm_count, cudaDevAttrMultiProcessorCount, h->h.ws.device);
    e = cudaMemset(static_cast<uint8_t*>(base) + workspace_zero_from(), 0, workspace_bytes() - workspace_zero_from());
    if (e != cudaSuccess) {
        set_last_error("qw3_ws_create: cudaMemset -> %s", cudaGetErrorString(e));
        cudaFree(base);
        delete h;
        return QW3_ERR_CUDA;
    }
    *out = h;
    return QW3_OK;
}

int qw3_ws_destroy(qw3_ws_t ws) {
    if (ws) {
        if (ws->h.ws.base) cudaFree(ws->h.ws.base);
        delete ws;
    }
    return QW3_OK;
}

int qw3_ws_set_pdl(qw3_ws_t ws, int enable) {
    QW3_REQUIRE(ws, "qw3_ws_set_pdl: null workspace");
    ws->h.use_pdl = enable ? 1 : 0;
    return QW3_OK;
}

int qw3_ws_check(qw3_ws_t ws, void* stream) {
    QW3_REQUIRE(ws, "qw3_ws_check: null workspace");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int err = 0;
    QW3_CUDA(cudaMemcpyAsync(&err, ws->h.ws.err, 4, cudaMemcpyDeviceToHost, st));
    QW3_CUDA(cudaStreamSynchronize(st));
    if (err != 0) {
        // Counters may be left mid-count by the kernel that gave up: start clean again.
        uint8_t* base = static_cast<uint8_t*>(ws->h.ws.base);
        if (base) QW3_CUDA(cudaMemsetAsync(base + workspace_zero_from(), 0, workspace_bytes() - workspace_zero_from(), st));
        else QW3_CUDA(cudaMemsetAsync(ws->h.ws.err, 0, 4, st));
        QW3_CUDA(cudaStreamSynchronize(st));
        set_last_error("a bounded device-side wait gave up (device error word = 0x%x)", err);
        return QW3_ERR_TIMEOUT;
    }
    return QW3_OK;
}

}  // extern "C"

namespace qw3 {

// Shared by the C entry point and the engine: validates, fills the parameter block, launches.
int gemv_launch(const W4Desc* d, const Qw3GemvArgs* a, const Workspace* ws, bool pdl, cudaStream_t st) {
    QW3_REQUIRE(d && a && ws, "qw3_gemv_w4a16: null argument");
    QW3_REQUIRE(a->d_x, "qw3_gemv_w4a16: d_x is null");
    QW3_REQUIRE(a->epilogue >= QW3_EPI_STORE && a->epilogue <= QW3_EPI_ARGMAX, "qw3_gemv_w4a16: unknown epilogue %d", a->epilogue);
    GemvParams p = {};
    p.scale = d->scale; p.zp = d->zp; p.n_alloc = (int)d->n_alloc;
    p.M = (int)d->M; p.K = (int)d->K; p.Mb = p.M / 128; p.Kb = p.K / 128;
    p.n_tiles = (p.M + TI - 1) / TI;
    p.upt = p.K / UNIT_ROWS;
    p.U = (long long)p.n_tiles * p.upt;
    p.x = static_cast<const __half*>(a->d_x);
    p.gamma = static_cast<const __half*>(a->d_gamma);
    p.eps = a->eps;
    p.epilogue = a->epilogue;
    p.y = static_cast<__half*>(a->d_y);
    p.ws = *ws;
    if (a->epilogue == QW3_EPI_ROPE_KV) {
        QW3_REQUIRE(a->d_y && a->d_k_cache && a->d_v_cache && a->d_cos && a->d_sin, "qw3_gemv_w4a16: ROPE_KV needs q, caches and tables");
        QW3_REQUIRE(a->head_dim == 128, "qw3_gemv_w4a16: head_dim must be 128");
        QW3_REQUIRE(p.M % 3 == 0 && (p.M / 3) == a->heads * 128, "qw3_gemv_w4a16: ROPE_KV needs out_dim = 3*heads*128");
        QW3_REQUIRE(a->d_pos || (a->pos >= 0 && a->pos < a->max_pos), "qw3_gemv_w4a16: pos out of range");
        p.kc = static_cast<__half*>(a->d_k_cache); p.vc = static_cast<__half*>(a->d_v_cache);
        p.cos_t = static_cast<const __half*>(a->d_cos); p.sin_t = static_cast<const __half*>(a->d_sin);
        p.hidden = p.M / 3; p.max_pos = a->max_pos; p.d_pos = a->d_pos; p.pos = a->pos;
    } else if (a->epilogue == QW3_EPI_ARGMAX) {
        QW3_REQUIRE(a->d_token, "qw3_gemv_w4a16: ARGMAX needs d_token");
        p.d_token = a->d_token; p.logits_f32 = a->d_logits_f32;
    } else {
        QW3_REQUIRE(a->d_y, "qw3_gemv_w4a16: d_y is null");
    }
    const bool uniform = d->uniform != 0;
    if (!uniform) {
        const int n_used = p.Kb < p.n_alloc ? p.Kb : p.n_alloc;
        QW3_REQUIRE(n_used <= MAX_GROUPS, "qw3_gemv_w4a16: more than %d distinct groups", MAX_GROUPS);
    }
    const size_t smem = gemv_smem_bytes(p.K, uniform);
    QW3_REQUIRE(smem <= 227 * 1024, "qw3_gemv_w4a16: in_dim=%d needs %zu bytes of shared memory", p.K, smem);
    int grid = ws->sm_count < WS_MAX_CTAS ? ws->sm_count : WS_MAX_CTAS;
    if ((long long)grid > p.U) grid = (int)p.U;
    if (uniform) {
        if (d->zp_integral) return launch_gemv<true, true>(d, p, grid, smem, pdl, st);
        return launch_gemv<true, false>(d, p, grid, smem, pdl, st);
    }
    if (d->zp_integral) return launch_gemv<false, true>(d, p, grid, smem, pdl, st);
    return launch_gemv<false, false>(d, p, grid, smem, pdl, st);
}

const W4Desc* w4_desc(qw3_w4_t w) { return &w->d; }
const Workspace* ws_struct(qw3_ws_t ws) { return &ws->h.ws; }
bool ws_pdl(qw3_ws_t ws) { return ws->h.use_pdl != 0; }

}  // namespace qw3

extern "C" int qw3_gemv_w4a16(qw3_w4_t w, const Qw3GemvArgs* args, qw3_ws_t ws, void* stream) {
    QW3_REQUIRE(w && ws, "qw3_gemv_w4a16: null descriptor or workspace");
    return gemv_launch(&w->d, args, &ws->h.ws, ws->h.use_pdl != 0, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the fused dequant-GEMV
// ------------------------------------------------------------------------------------------------
// Some callers must not allocate device memory when they run an operator: a serving process that
// reserved its whole memory budget at start-up and hands out slices from its own pool, a plug-in
// called from inside another framework's execution step (where cudaMalloc would synchronise the
// device and stall every other stream), or code that is simply forbidden to grow the process.
// qw3_gemv_w4a16 needs a qw3_ws_t workspace (one cudaMalloc) and a qw3_w4_t descriptor (host
// memory).  The entry point below needs neither: its split-K scratch lives in a fixed array that is
// part of the library image on every GPU that loads it, and the matrix is described by plain
// arguments.  The price is a size limit and one shared scratch area per GPU.
namespace qw3 {

constexpr int NOALLOC_MAX_DIM = 16384;                          // largest out_dim and in_dim accepted
constexpr int NOALLOC_MAX_TILES = NOALLOC_MAX_DIM / TI;         // 16
constexpr size_t NOALLOC_PARTIAL_BYTES = (size_t)(WS_MAX_CTAS + NOALLOC_MAX_TILES) * TI * 4;   // 1,114,112
constexpr size_t NOALLOC_TAIL_BYTES = 1024;                     // arrival counters, error word
constexpr size_t NOALLOC_BYTES = NOALLOC_PARTIAL_BYTES + NOALLOC_TAIL_BYTES;                   // ~1.06 MiB per GPU

// Held by every GPU that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

struct NoAllocDevice {
    void* base = nullptr;   // device address of g_noalloc_scratch on this device
    int sm_count = 0;
    bool ready = false;
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mutex;

// Once per device, with that device current: in host code the array's name is only a handle, the
// address a kernel can use comes from cudaGetSymbolAddress.
static int noalloc_setup(int dev, NoAllocDevice** out) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& d = g_noalloc_dev[dev];
    if (!d.ready) {
        void* ptr = nullptr;
        QW3_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        QW3_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        const int rc = gemv_init_device();   // shared-memory opt-in of the kernel: an attribute, not an allocation
        if (rc != QW3_OK) return rc;
        d.base = ptr;
        d.ready = true;
    }
    *out = &d;
    return QW3_OK;
}

}  // namespace qw3

extern "C" int qw3_gemv_w4a16_noalloc(const void* d_packed, const void* d_scale, const void* d_zp, int64_t n_groups_alloc,
                                      int64_t out_dim, int64_t in_dim, int zp_integral, const void* d_x, void* d_y,
                                      void* stream) {
    QW3_REQUIRE(d_packed && d_scale && d_zp && d_x && d_y, "qw3_gemv_w4a16_noalloc: null pointer");
    QW3_REQUIRE(out_dim > 0 && in_dim > 0 && out_dim % 128 == 0 && in_dim % 128 == 0,
                "qw3_gemv_w4a16_noalloc: out_dim=%lld and in_dim=%lld must be positive multiples of 128",
                (long long)out_dim, (long long)in_dim);
    QW3_REQUIRE(out_dim <= NOALLOC_MAX_DIM && in_dim <= NOALLOC_MAX_DIM,
                "qw3_gemv_w4a16_noalloc: out_dim=%lld, in_dim=%lld exceed the fixed scratch (at most %d each); "
                "use qw3_gemv_w4a16 with a workspace for larger matrices",
                (long long)out_dim, (long long)in_dim, NOALLOC_MAX_DIM);
    QW3_REQUIRE(n_groups_alloc > 0 && n_groups_alloc <= 0x7fffffff, "qw3_gemv_w4a16_noalloc: n_groups_alloc out of range");
    QW3_REQUIRE((reinterpret_cast<uintptr_t>(d_packed) & 15) == 0, "qw3_gemv_w4a16_noalloc: packed pointer must be 16-byte aligned");
    int dev = 0;
    QW3_CUDA(cudaGetDevice(&dev));
    QW3_REQUIRE(dev >= 0 && dev < 64, "qw3_gemv_w4a16_noalloc: device index %d not supported", dev);
    NoAllocDevice* nd = nullptr;
    {
        const int rc = noalloc_setup(dev, &nd);
        if (rc != QW3_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    W4Desc d = {};
    d.packed = static_cast<const uint8_t*>(d_packed);
    d.scale = static_cast<const __half*>(d_scale);
    d.zp = static_cast<const __half*>(d_zp);
    d.n_alloc = n_groups_alloc; d.M = out_dim; d.K = in_dim; d.zp_integral = zp_integral ? 1 : 0;
    const int64_t Mb = out_dim / 128, Kb = in_dim / 128;
    d.uniform = (Mb % Kb == 0) || (Kb % n_groups_alloc == 0 && Mb % n_groups_alloc == 0);
    {
        const int rc = encode_2d_u32(&d.tmap, d_packed, (uint64_t)out_dim / 8, (uint64_t)in_dim, (uint64_t)out_dim / 2,
                                     TI / 8, UNIT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != QW3_OK) return rc;
    }
    uint8_t* base = static_cast<uint8_t*>(nd->base);
    Workspace ws = {};
    ws.partials = reinterpret_cast<float*>(base);
    ws.counters = reinterpret_cast<int32_t*>(base + NOALLOC_PARTIAL_BYTES);          // [NOALLOC_MAX_TILES]
    ws.tiles_done = reinterpret_cast<int32_t*>(base + NOALLOC_PARTIAL_BYTES + 256);
    ws.err = reinterpret_cast<int32_t*>(base + NOALLOC_PARTIAL_BYTES + 512);
    ws.device = dev;
    ws.sm_count = nd->sm_count;
    // The array keeps whatever the previous call left: the arrival counters must start at zero (the partial
    // sums are always written before they are read).  The error word behind them is NOT cleared here: a bounded
    // wait that gave up stays recorded until qw3_gemv_w4a16_noalloc_status reads it.
    QW3_CUDA(cudaMemsetAsync(base + NOALLOC_PARTIAL_BYTES, 0, 512, st));
    Qw3GemvArgs a;
    std::memset(&a, 0, sizeof(a));
    a.d_x = d_x;
    a.d_y = d_y;
    a.epilogue = QW3_EPI_STORE;
    return gemv_launch(&d, &a, &ws, false, st);
}

// The error word of the fixed scratch: QW3_ERR_TIMEOUT when a bounded wait of an earlier qw3_gemv_w4a16_noalloc call
// on this GPU gave up (its output is then void), QW3_OK otherwise.  Reads and clears the word; synchronises `stream`;
// allocates nothing (the word is copied into a local variable).
extern "C" int qw3_gemv_w4a16_noalloc_status(void* stream) {
    int dev = 0;
    QW3_CUDA(cudaGetDevice(&dev));
    QW3_REQUIRE(dev >= 0 && dev < 64, "qw3_gemv_w4a16_noalloc_status: device index %d not supported", dev);
    NoAllocDevice* nd = nullptr;
    {
        const int rc = noalloc_setup(dev, &nd);
        if (rc != QW3_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* word = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(nd->base) + NOALLOC_PARTIAL_BYTES + 512);
    int err = 0;
    QW3_CUDA(cudaMemcpyAsync(&err, word, 4, cudaMemcpyDeviceToHost, st));
    QW3_CUDA(cudaStreamSynchronize(st));
    if (err != 0) {
        QW3_CUDA(cudaMemsetAsync(word, 0, 4, st));
        QW3_CUDA(cudaStreamSynchronize(st));
        set_last_error("a bounded device-side wait of qw3_gemv_w4a16_noalloc gave up (device error word = 0x%x)", err);
        return QW3_ERR_TIMEOUT;
    }
    return QW3_OK;
}
