// Tensor-core W4A16 contraction for several activation rows (prefill / batched rows) on sm_100a:
//   Y[r][i] = sum_j W(i, j) * X[r][j],   W(i, j) = hmul(hsub(half(q), zp[g]), scale[g])  (bit-exact),
// with tcgen05.mma (fp16 x fp16 -> fp32 in tensor memory).  The reference has no batched path: it
// feeds prompts token by token through cublasGemmEx at n = 1 (Inference.cu:1304-1343, 1052-1065);
// this is the same product for `rows` tokens at once.
//
// One CTA computes a tile of 128 outputs x N rows of X (N = 16..256).  Nineteen warps:
//   warp 0      TMA producer: per 64-deep K block one box of activations [N][64] (128-byte swizzle, K-major
//               operand B)
//   warp 1, 18  MMA issuers (one lane each; even / odd K blocks into separate accumulators in tensor memory, which
//               warp 1 allocates), tcgen05.commit frees the stages
//   warps 2..17 read the packed nibbles of the tile straight from global memory (16 bytes per thread and row, one
//               K block ahead; four groups of four warps take the K blocks in turn), unpack them to fp16 with
//               the reference's two roundings and write operand A to shared memory in the MN-major 128-byte-swizzled canonical layout (outputs are
//               contiguous in the packed stream, so MN-major needs no transposition); afterwards the
//               same warps read the accumulators back (tcgen05.ld) and store Y as fp16.
// Within every group of 8 outputs the rows of A are stored in the order the lop3 unpack yields them
// (0,4,1,5,2,6,3,7); the epilogue undoes that permutation when it computes the output index.
// All mbarrier waits are bounded; a wait that gives up sets the workspace error word.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace qw3 {

const Workspace* ws_struct(qw3_ws_t ws);
const W4Desc* w4_desc(qw3_w4_t w);

constexpr int GM_TILE_M = 128;                 // outputs per CTA
constexpr int GM_BK = 64;                      // K per pipeline stage
constexpr int GM_A_BYTES = GM_TILE_M * GM_BK * 2;        // 16384
constexpr int GM_MAX_STAGES = 24;              // mbarrier slots per ring
// Operand A (16 KB per K block, unpacked) and the activations share one ring depth and ONE release barrier per
// stage: a tcgen05.commit costs the issuing lane ~150 ns, so a K block gets a single commit.  The depth is a template
// parameter (6, or 4 with 256-row tiles).
constexpr int GM_UNPACK_WARPS = 16;           // unpack / epilogue warps: four groups of four, taking K blocks in turn
                                              // (an unpack warp is latency-bound on its own chain: more groups, more K blocks in flight)
constexpr int GM_ISSUER_B = 2 + GM_UNPACK_WARPS;   // warp index of the second MMA issuer
constexpr int GM_THREADS = 32 * (GM_ISSUER_B + 1);

struct GemmParams {
    const uint8_t* packed;   // [K][M/2] bytes; the unpack warps read their 16-byte pieces straight from global memory
    const __half* scale;
    const __half* zp;
    int n_alloc, M, K, Mb, Kb;
    int uniform, exact;
    int rows;          // rows of X / Y
    int n_tile;        // UMMA N: 16..256, multiple of 16
    int tmem_cols;     // power of two >= n_acc * acc_stride
    int n_acc;         // accumulators in tensor memory (2 or 4, half per MMA issuer): the MMAs of a K block go to different ones, so
                       // that they do not wait for each other (an MMA into the same accumulator is ~240 cycles
                       // behind the one before, whatever N); the epilogue adds them in a fixed order
    int acc_stride;    // columns between accumulators
    __half* y;         // [rows][M]
    int epilogue;      // QW3_EPI_STORE, QW3_EPI_RESIDUAL (y = hadd(y, result), Inference.cu:1145-1156) or QW3_EPI_GELU
                       // (Inference.cu:271-279): what the batched prompt phase needs after wo / w2 and after w1
    float* part;       // split-K: fp32 partial products [splits][rows][M] (null: one split, y is written directly)
    int* err;
    int a_lbo, a_sbo, a_kstep;   // operand A descriptor: byte offsets between 64-output blocks, between 8-deep K blocks, per K=16 step
};

__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred;
}

// Shared-memory matrix descriptor (tcgen05): start >> 4 in bits 0-13, leading byte offset >> 4 in
// bits 16-29, stride byte offset >> 4 in bits 32-45, version 1 in bits 46-47, swizzle mode in bits 61-63
// (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One output element: fp32 sum -> fp16, then the epilogue in fp16 as the decode path does it.
__device__ __forceinline__ __half gemm_epilogue(float v, int epilogue, __half old) {
    const __half h = __float2half_rn(v);
    if (epilogue == QW3_EPI_RESIDUAL) return h_add(old, h);
    if (epilogue == QW3_EPI_GELU) return gelu_h(h);
    return h;
}

template <int GM_STAGES>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int x_bytes = p.n_tile * 128;                                   // [n_tile][64] fp16
    static_assert(GM_STAGES <= GM_MAX_STAGES && GM_STAGES >= GM_UNPACK_WARPS / 4, "ring depth");
    constexpr int GM_A_STAGES = GM_STAGES, GM_X_STAGES = GM_STAGES;
    uint8_t* a_st = smem;                                                 // GM_A_STAGES x 16 KB (1024-aligned)
    uint8_t* x_st = smem + GM_A_STAGES * GM_A_BYTES;                      // GM_X_STAGES x x_bytes (multiple of 1024)
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_st + GM_X_STAGES * x_bytes);
    const uint32_t a_full = smem_u32(bars + 2 * GM_MAX_STAGES), a_empty = smem_u32(bars + 3 * GM_MAX_STAGES);
    const uint32_t x_full = smem_u32(bars + 4 * GM_MAX_STAGES), x_empty = a_empty;   // one release barrier per stage
    const uint32_t acc_full = smem_u32(bars + 6 * GM_MAX_STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 * GM_MAX_STAGES + 1);
    int* s_dead = reinterpret_cast<int*>(tmem_slot + 1);   // bars: (6 * 24 + 2) * 8 bytes < 1280

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y;
    // split-K: grid.z CTAs share the K blocks of a tile; each handles [kb_lo, kb_lo + n_kb)
    const int n_kb_all = p.K / GM_BK;
    const int kb_lo = (int)((long long)blockIdx.z * n_kb_all / gridDim.z);
    const int n_kb = (int)((long long)(blockIdx.z + 1) * n_kb_all / gridDim.z) - kb_lo;

    if (tid == 0) {
        for (int s = 0; s < GM_X_STAGES; ++s) {
            mbar_init(x_full + 8 * s, 1);
        }
        for (int s = 0; s < GM_A_STAGES; ++s) {
            mbar_init(a_full + 8 * s, 4);       // the 4 unpack warps of the group that owns the K block
            mbar_init(a_empty + 8 * s, 1);      // commit of the MMAs that read A and X of the stage
        }
        mbar_init(acc_full, 2);             // the last commit of each of the two MMA issuers
        *s_dead = 0;
        mbar_fence_init();
    }
    if (warp == 1) {   // tensor memory for the accumulators: 128 lanes x tmem_cols 32-bit columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer of the activations ------------------------------------------
        // (the packed nibbles do not go through TMA: a 128-output tile is 64 bytes wide, and a box of 64 such rows
        // cost the copy engine more per K block than everything else in the CTA)
        if (lane == 0) {
            tma_prefetch_desc(&tmap_x);
            bool ok = true;
            for (int kb = 0; kb < n_kb && ok; ++kb) {
                const int s = kb % GM_X_STAGES;
                if (kb >= GM_X_STAGES) ok = mbar_wait(x_empty + 8 * s, ((kb / GM_X_STAGES) - 1) & 1);   // freed by the MMAs' commit
                if (!ok) break;
                mbar_expect_tx(x_full + 8 * s, (uint32_t)x_bytes);
                tma_load_2d(smem_u32(x_st + s * x_bytes), &tmap_x, (kb_lo + kb) * GM_BK, tile_n * p.n_tile, x_full + 8 * s);
            }
            if (!ok) {
                atomicCAS(p.err, 0, 0x30001);
                *s_dead = 1;
            }
        }
    } else if (warp == 1 || warp == GM_ISSUER_B) {
        // ---------------- MMA issuers ------------------------------------------------------------
        // The instruction chain of an issuing lane (two barrier waits, four MMAs, one commit: ~900 cycles) is what a
        // K block costs a CTA when the row tile is small, so TWO warps issue: warp 1 takes the even K blocks, the
        // last warp the odd ones, each into its own accumulators (summed by the epilogue).  One lane per warp runs
        // the loop; ring indices and phases are running counters, descriptors a constant plus additions.
        if (lane == 0) {
            const int who = warp == 1 ? 0 : 1;
            // instruction descriptor: D = f32, A = B = f16, A MN-major (bit 15), B K-major, N >> 3, M >> 4
            const uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(p.n_tile >> 3) << 17) | ((uint32_t)(GM_TILE_M >> 4) << 24);
            const uint64_t adesc0 = make_smem_desc(smem_u32(a_st), p.a_lbo, p.a_sbo);
            const uint64_t bdesc0 = make_smem_desc(smem_u32(x_st), 16, 1024);
            const uint32_t a_step = (uint32_t)(p.a_kstep >> 4), a_stage = (uint32_t)(GM_A_BYTES >> 4), x_stage = (uint32_t)(x_bytes >> 4);
            const int half_acc = p.n_acc >> 1;                        // accumulators of this issuer
            const uint32_t my_tmem = tmem_base + (uint32_t)(who * half_acc * p.acc_stride);
            int s = who;                                              // stage of K block `who` (GM_STAGES >= 2)
            uint32_t phase = 0;
            bool first = true;
            for (int kb = who; kb < n_kb; kb += 2) {
                if (*s_dead != 0) break;
                if (!(mbar_wait(x_full + 8 * s, phase) && mbar_wait(a_full + 8 * s, phase))) {
                    atomicCAS(p.err, 0, 0x30002);
                    *s_dead = 1;
                    break;
                }
                // A (MN-major): 64-output blocks 8 KB apart (LBO), 8-deep K blocks 1 KB apart (SBO); K=16 = 2 blocks
                // B (K-major): 8-row groups 1 KB apart (SBO); K=16 = 32 bytes inside the swizzled row
                const uint64_t adesc = adesc0 + (uint64_t)((uint32_t)s * a_stage);
                const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)s * x_stage);
#pragma unroll
                for (int ks = 0; ks < GM_BK / 16; ++ks) {
                    const int acc = ks & (half_acc - 1);
                    umma_f16(my_tmem + (uint32_t)(acc * p.acc_stride), adesc + (uint64_t)(ks * a_step), bdesc + (uint64_t)(ks * 2), idesc,
                             (!first || ks >= half_acc) ? 1u : 0u);
                }
                first = false;
                umma_commit(a_empty + 8 * s);    // A and X of the stage are free once these MMAs have read them
                if (kb + 2 >= n_kb) umma_commit(acc_full);   // this issuer's last K block
                s += 2;
                if (s >= GM_STAGES) { s -= GM_STAGES; phase ^= 1u; }
            }
            // Drain: the release arrivals of this issuer's last K blocks are waited for by nobody else (no later block
            // reuses those stages).  They must have landed before the CTA exits, or they would hit the barriers of
            // the next CTA that gets this shared memory.
            for (int kb = who; kb < n_kb; kb += 2) {
                if (kb + GM_STAGES < n_kb || *s_dead != 0) continue;
                if (!mbar_wait(a_empty + 8 * (kb % GM_STAGES), (uint32_t)(kb / GM_STAGES) & 1u)) {
                    atomicCAS(p.err, 0, 0x30006);
                    *s_dead = 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- unpack warps (2..17), then epilogue -----------------------------------
        const int grp = (warp - 2) >> 2;          // group g unpacks the K blocks g, g + 4, ...
        const int ut = (tid - 64) & 127;          // 0..127 inside the group
        const int c4 = ut & 3, krow = ut >> 2;    // 16-byte chunk (32 outputs) of a row; row 0..31 (+32)
        const int ib = tile_m;                    // the tile is exactly one block of 128 outputs
        const int ibk = ib % p.Kb;
        DqConst ku = {0u, 0u, 0u};
        if (p.uniform) {
            const int g = ibk % p.n_alloc;
            ku = p.exact ? make_const<true>(p.zp[g], p.scale[g]) : make_const<false>(p.zp[g], p.scale[g]);
        }
        bool dead = false;
        // this thread's two 16-byte pieces of a K block (rows krow and krow + 32), requested two own blocks ahead
        const size_t pitch = (size_t)p.M / 2;
        const uint8_t* gsrc = p.packed + (size_t)tile_m * (GM_TILE_M / 2) + c4 * 16;
        auto request = [&](const int kb, uint4 (&dst)[2]) {
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                const size_t row = (size_t)(kb_lo + kb) * GM_BK + krow + pass * 32;
                dst[pass] = kb < n_kb ? __ldg(reinterpret_cast<const uint4*>(gsrc + row * pitch)) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        uint4 nxt[2], nxt2[2];   // two own K blocks in flight
        request(grp, nxt);
        request(grp + GM_UNPACK_WARPS / 4, nxt2);
        for (int kb = grp; kb < n_kb && !dead; kb += GM_UNPACK_WARPS / 4) {
            const int t = kb % GM_A_STAGES;
            const uint4 cur[2] = {nxt[0], nxt[1]};
            nxt[0] = nxt2[0];
            nxt[1] = nxt2[1];
            request(kb + 2 * (GM_UNPACK_WARPS / 4), nxt2);
            if (kb >= GM_A_STAGES && !mbar_wait(a_empty + 8 * t, ((kb / GM_A_STAGES) - 1) & 1)) {
                if (lane == 0) atomicCAS(p.err, 0, 0x30003);
                *s_dead = 1;
                dead = true;
                break;
            }
            uint8_t* adst = a_st + t * GM_A_BYTES + (c4 >> 1) * 8192;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                const int k = krow + pass * 32;
                const uint4 raw = cur[pass];
                DqConst kc = ku;
                if (!p.uniform) {
                    const long long j = (long long)(kb_lo + kb) * GM_BK + k;
                    int g = ibk + (int)((j * p.Mb) % p.Kb);
                    g -= g >= p.Kb ? p.Kb : 0;
                    g %= p.n_alloc;
                    kc = p.exact ? make_const<true>(p.zp[g], p.scale[g]) : make_const<false>(p.zp[g], p.scale[g]);
                }
                const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
                uint8_t* rowp = adst + (k >> 3) * 1024 + (k & 7) * 128;
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    uint32_t lo0, hi0, lo1, hi1;
                    if (p.exact) {
                        dq_pair<true>(w4[wd], kc, lo0, hi0);
                        dq_pair<true>(w4[wd] >> 8, kc, lo1, hi1);
                    } else {
                        dq_pair<false>(w4[wd], kc, lo0, hi0);
                        dq_pair<false>(w4[wd] >> 8, kc, lo1, hi1);
                    }
                    const int chunk = 4 * (c4 & 1) + wd;   // 8 outputs, stored in unpack order (0,4,1,5,2,6,3,7)
                    *reinterpret_cast<uint4*>(rowp + ((chunk ^ (k & 7)) << 4)) = make_uint4(lo0, hi0, lo1, hi1);
                }
            }
            // generic-proxy writes of A must be visible to the tensor core (async proxy) before the arrive
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full + 8 * t);
        }
        // ---------------- epilogue: accumulators -> fp16 Y ----------------------------------------
        if (!dead && *s_dead == 0 && !mbar_wait(acc_full, 0)) {
            if (lane == 0) atomicCAS(p.err, 0, 0x30004);
            *s_dead = 1;
            dead = true;
        }
        if (!dead && *s_dead == 0) {
            tc_fence_after();
            const int q = warp & 3;                           // TMEM lanes 32q..32q+31 belong to this warp
            const int m = 32 * q + lane;                      // row of A = TMEM lane
            const int pos = m & 7;                            // position inside the 8-group, in unpack order
            const int nib = (pos >> 1) + ((pos & 1) << 2);    // 0,4,1,5,2,6,3,7
            const int i = tile_m * GM_TILE_M + (m & ~7) + nib;
            // the warps of a lane quarter take the 16-column groups in turn
            for (int c0 = 16 * ((warp - 2) >> 2); c0 < p.n_tile; c0 += 16 * (GM_UNPACK_WARPS / 4)) {
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
                float f[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[e]);
                for (int acc = 1; acc < p.n_acc; ++acc) {   // fixed order: accumulator 0 + 1 + 2 + 3
                    tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(acc * p.acc_stride + c0), v);
#pragma unroll
                    for (int e = 0; e < 16; ++e) f[e] += __uint_as_float(v[e]);
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int r = tile_n * p.n_tile + c0 + e;
                    if (r < p.rows) {
                        if (p.part != nullptr) p.part[((size_t)blockIdx.z * p.rows + r) * p.M + i] = f[e];
                        else {
                            __half* dst = p.y + (size_t)r * p.M + i;
                            *dst = gemm_epilogue(f[e], p.epilogue, p.epilogue == QW3_EPI_RESIDUAL ? *dst : __half());
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

// Split-K: sums the fp32 partial products of the splits in split order and rounds once to fp16.
__global__ void gemm_splitk_reduce_kernel(const float* __restrict__ part, int splits, long long n, int epilogue, __half* y) {
    const long long i = 2 * ((long long)blockIdx.x * blockDim.x + threadIdx.x);
    if (i >= n) return;
    float2 acc = *reinterpret_cast<const float2*>(part + i);
    for (int z = 1; z < splits; ++z) {
        const float2 v = *reinterpret_cast<const float2*>(part + (size_t)z * n + i);
        acc.x += v.x;
        acc.y += v.y;
    }
    const __half2 old = epilogue == QW3_EPI_RESIDUAL ? *reinterpret_cast<const __half2*>(y + i) : __half2();
    *reinterpret_cast<__half2*>(y + i) =
        __halves2half2(gemm_epilogue(acc.x, epilogue, __low2half(old)), gemm_epilogue(acc.y, epilogue, __high2half(old)));
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
        return QW3_ERR_CUDA;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return QW3_ERR_CUDA;
    }
    return QW3_OK;
}

}  // namespace qw3

using namespace qw3;

namespace qw3 {
int gemm_launch(qw3_w4_t w, const void* d_x, int64_t rows, void* d_y, qw3_ws_t ws, void* stream, int epilogue);
}

extern "C" int qw3_gemm_w4a16(qw3_w4_t w, const void* d_x, int64_t rows, void* d_y, qw3_ws_t ws, void* stream) {
    return qw3::gemm_launch(w, d_x, rows, d_y, ws, stream, QW3_EPI_STORE);
}

// The contraction with an optional epilogue (the engine's batched prompt phase fuses the residual add and the GeLU).
int qw3::gemm_launch(qw3_w4_t w, const void* d_x, int64_t rows, void* d_y, qw3_ws_t ws, void* stream, int epilogue) {
    QW3_REQUIRE(w && d_x && d_y && ws, "qw3_gemm_w4a16: null argument");
    QW3_REQUIRE(epilogue == QW3_EPI_STORE || epilogue == QW3_EPI_RESIDUAL || epilogue == QW3_EPI_GELU, "qw3_gemm_w4a16: epilogue");
    QW3_REQUIRE(rows >= 1 && rows <= (1 << 20), "qw3_gemm_w4a16: rows out of range");
    QW3_REQUIRE((reinterpret_cast<uintptr_t>(d_x) & 15) == 0, "qw3_gemm_w4a16: X must be 16-byte aligned");
    const W4Desc* d = w4_desc(w);
    GemmParams p = {};
    p.packed = d->packed;
    p.scale = d->scale; p.zp = d->zp; p.n_alloc = (int)d->n_alloc;
    p.M = (int)d->M; p.K = (int)d->K; p.Mb = p.M / 128; p.Kb = p.K / 128;
    p.uniform = d->uniform; p.exact = d->zp_integral;
    p.rows = (int)rows;
    p.n_tile = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    p.n_acc = p.n_tile <= 64 ? 4 : 2;       // half of them per MMA issuer
    p.acc_stride = p.n_tile < 32 ? 32 : p.n_tile;
    p.tmem_cols = p.n_acc * p.acc_stride;   // 128, 128, 256, 256, 512 columns: powers of two
    p.y = static_cast<__half*>(d_y);
    p.epilogue = epilogue;
    p.err = ws_struct(ws)->err;
    p.a_lbo = 8192; p.a_sbo = 1024; p.a_kstep = 2048;
    CUtensorMap tmap_x;
    int rc;
    rc = encode_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, d_x, (uint64_t)d->K, (uint64_t)rows, (uint64_t)d->K * 2, GM_BK,
                   (uint32_t)p.n_tile, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != QW3_OK) return rc;
    // shared memory per stage: 16 KB of operand A + n_tile x 128 bytes of activations; 6 stages (4 with 256-row tiles)
    const int stages = p.n_tile <= 128 ? 6 : 4;
    const size_t smem = (size_t)stages * (GM_A_BYTES + p.n_tile * 128) + 1280;
    static std::once_flag attr_once[16];
    int dev = 0;
    QW3_CUDA(cudaGetDevice(&dev));
    if (dev < 16)
        std::call_once(attr_once[dev], [] {
            cudaFuncSetAttribute(gemm_w4a16_tc_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            cudaFuncSetAttribute(gemm_w4a16_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        });
    // Few rows and few output tiles leave most SMs without a CTA: split K over grid.z (fp32 partial products in the
    // workspace, summed in split order by a second kernel) until ~one CTA per SM, while the partials fit.
    const long long ctas = (d->M / GM_TILE_M) * ((rows + p.n_tile - 1) / p.n_tile);
    const long long part_cap = (long long)(WS_MAX_CTAS + WS_MAX_TILES) * WS_TILE;   // floats in the workspace
    int splits = 1;
    while (splits < 8 && ctas * (splits * 2) <= ws_struct(ws)->sm_count && (p.K / GM_BK) / (splits * 2) >= 8 &&
           (long long)(splits * 2) * rows * d->M <= part_cap)
        splits *= 2;
    p.part = splits > 1 ? ws_struct(ws)->partials : nullptr;
    dim3 grid((unsigned)(d->M / GM_TILE_M), (unsigned)((rows + p.n_tile - 1) / p.n_tile), (unsigned)splits);
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (stages == 6)
        gemm_w4a16_tc_kernel<6><<<grid, GM_THREADS, smem, st>>>(tmap_x, p);
    else
        gemm_w4a16_tc_kernel<4><<<grid, GM_THREADS, smem, st>>>(tmap_x, p);
    QW3_CUDA(cudaGetLastError());
    if (splits > 1) {
        const long long n = rows * d->M;
        gemm_splitk_reduce_kernel<<<(unsigned)((n / 2 + 255) / 256), 256, 0, st>>>(p.part, splits, n, p.epilogue, p.y);
        QW3_CUDA(cudaGetLastError());
    }
    return QW3_OK;
}
