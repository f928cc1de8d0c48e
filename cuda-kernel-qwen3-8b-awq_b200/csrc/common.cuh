// Shared device helpers for the sm_100a kernels: status plumbing, explicitly rounded fp16
// arithmetic, mbarrier / TMA / mma / programmatic-dependent-launch PTX wrappers.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qw3_cabi.h"

namespace qw3 {

// ---- host-side status plumbing ---------------------------------------------------------------
void set_last_error(const char* fmt, ...);

#define QW3_CUDA(expr)                                                                         \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess) {                                                              \
            ::qw3::set_last_error("%s:%d: %s -> %s", __FILE__, __LINE__, #expr,                \
                                  cudaGetErrorString(e__));                                    \
            return QW3_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

#define QW3_REQUIRE(cond, ...)                                                                 \
    do {                                                                                       \
        if (!(cond)) {                                                                         \
            ::qw3::set_last_error(__VA_ARGS__);                                                \
            return QW3_ERR_ARG;                                                                \
        }                                                                                      \
    } while (0)

// Workspace: scratch of the split-K fix-up, attention partials, arg-max partials, error word.
constexpr int WS_TILE = 1024;          // outputs per GEMV tile
constexpr int WS_MAX_CTAS = 256;       // upper bound on the GEMV grid
constexpr int WS_MAX_TILES = 2048;     // upper bound on out_dim / WS_TILE
constexpr int WS_ATT_MAX_HEADS = 128;
constexpr int WS_ATT_MAX_SPLITS = 32;
constexpr int WS_ATT_STRIDE = 132;     // head_dim (128) outputs + running max + running sum + pad

struct Workspace {
    float*    partials;     // [(WS_MAX_CTAS + WS_MAX_TILES)][WS_TILE]
    int32_t*  counters;     // [WS_MAX_TILES] fix-up arrivals per tile (self-resetting)
    int32_t*  tiles_done;   // [1] arg-max arrivals (self-resetting)
    float*    arg_val;      // [WS_MAX_TILES]
    int32_t*  arg_idx;      // [WS_MAX_TILES]
    float*    att_part;     // [WS_ATT_MAX_HEADS][WS_ATT_MAX_SPLITS][WS_ATT_STRIDE]
    int32_t*  att_count;    // [WS_ATT_MAX_HEADS] (self-resetting)
    int32_t*  err;          // [1] device error word (0 = none)
    void*     base;         // single allocation backing all of the above (NULL for static scratch)
    int       device;
    int       sm_count;
};
size_t workspace_bytes();
void   workspace_carve(Workspace* ws, void* base);

// Descriptor of one quantised matrix (host memory only).
struct W4Desc {
    const uint8_t* packed;
    const __half*  scale;
    const __half*  zp;
    int64_t n_alloc, M, K;
    int     zp_integral;
    int     uniform;        // group of (i, j) does not depend on j
    CUtensorMap tmap;       // uint32 [K][M/8], box [8][128]
};

#ifdef __CUDACC__

// ---- explicitly rounded fp16 arithmetic (never contracted into fma) --------------------------
__device__ __forceinline__ __half h_add(__half a, __half b) {
    __half r;
    asm("add.rn.f16 %0, %1, %2;" : "=h"(*reinterpret_cast<unsigned short*>(&r))
        : "h"(*reinterpret_cast<unsigned short*>(&a)), "h"(*reinterpret_cast<unsigned short*>(&b)));
    return r;
}
__device__ __forceinline__ __half h_sub(__half a, __half b) {
    __half r;
    asm("sub.rn.f16 %0, %1, %2;" : "=h"(*reinterpret_cast<unsigned short*>(&r))
        : "h"(*reinterpret_cast<unsigned short*>(&a)), "h"(*reinterpret_cast<unsigned short*>(&b)));
    return r;
}
__device__ __forceinline__ __half h_mul(__half a, __half b) {
    __half r;
    asm("mul.rn.f16 %0, %1, %2;" : "=h"(*reinterpret_cast<unsigned short*>(&r))
        : "h"(*reinterpret_cast<unsigned short*>(&a)), "h"(*reinterpret_cast<unsigned short*>(&b)));
    return r;
}
__device__ __forceinline__ __half h_fma(__half a, __half b, __half c) {
    __half r;
    asm("fma.rn.f16 %0, %1, %2, %3;" : "=h"(*reinterpret_cast<unsigned short*>(&r))
        : "h"(*reinterpret_cast<unsigned short*>(&a)), "h"(*reinterpret_cast<unsigned short*>(&b)),
          "h"(*reinterpret_cast<unsigned short*>(&c)));
    return r;
}
// Interleaved-pair rotation of applyRotaryKernel (Inference.cu:172-173) as the reference's build executes it: the
// intrinsics emit mul.f16 / sub.f16 / add.f16 without a rounding modifier and the compiler contracts the first
// product of each line into the add; the second product keeps its own rounding.  Bit-equal to the compiled kernel.
__device__ __forceinline__ void rope_pair(__half x0, __half x1, __half cs, __half sn, __half& o0, __half& o1) {
    o0 = h_fma(x0, cs, __hneg(h_mul(x1, sn)));
    o1 = h_fma(x0, sn, h_mul(x1, cs));
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;  // (a & mask) | orv
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}
__device__ __forceinline__ uint32_t dup_h2(__half v) { return pack_h2(v, v); }

// One dequantised weight with the reference's two roundings (Inference.cu:102-104).
__device__ __forceinline__ __half dequant_one(uint32_t q, __half z, __half s) {
    return h_mul(h_sub(__int2half_rn((int)q), z), s);
}

// ---- AWQ unpack shared by the GEMV kernels -----------------------------------------------------
struct DqConst {  // per-group constants, duplicated into both halves
    uint32_t z;   // exact path: 1024 + zp;  generic path: zp
    uint32_t hz;  // exact path: -(64 + zp)
    uint32_t s;
};

template <bool EXACT>
__device__ __forceinline__ DqConst make_const(__half z, __half s) {
    DqConst c;
    if (EXACT) {
        c.z = dup_h2(h_add(__ushort_as_half(0x6400), z));   // 1024 + zp, exact for integral zp
        c.hz = dup_h2(h_sub(__ushort_as_half(0xD400), z));  // -64 - zp, exact
    } else {
        c.z = dup_h2(z);
        c.hz = 0;
    }
    c.s = dup_h2(s);
    return c;
}

// Eight nibbles of one row -> after `u = w` / `u = w >> 8`: two registers of dequantised pairs.
//   lo: nibbles (0,4) resp. (2,6);  hi: nibbles (1,5) resp. (3,7).
// Both roundings of the reference are kept: d = RN(q - zp), w = RN(d * scale).
template <bool EXACT>
__device__ __forceinline__ void dq_pair(uint32_t u, const DqConst& c, uint32_t& wlo, uint32_t& whi) {
    const uint32_t lo = lop3_and_or(u, 0x000f000fu, 0x64006400u);  // (1024 + q) x2
    const uint32_t hi = lop3_and_or(u, 0x00f000f0u, 0x64006400u);  // (1024 + 16 q) x2
    uint32_t dlo, dhi;
    if (EXACT) {
        dlo = h2_sub(lo, c.z);                     // (1024+q) - (1024+zp): exact operands, one rounding
        dhi = h2_fma(hi, 0x2C002C00u, c.hz);       // (1024+16q)/16 - (64+zp), one rounding
    } else {
        dlo = h2_sub(h2_sub(lo, 0x64006400u), c.z);                  // q exactly, then RN(q - zp)
        dhi = h2_sub(h2_fma(hi, 0x2C002C00u, 0xD400D400u), c.z);
    }
    wlo = h2_mul(dlo, c.s);
    whi = h2_mul(dhi, c.s);
}

// CTA that owns unit u when U units are cut into G equal contiguous ranges [c*U/G, (c+1)*U/G).
__device__ __forceinline__ int owner_of(long long u, int G, long long U) { return (int)(((u + 1) * G - 1) / U); }

// Arg-max order: larger value wins, equal values go to the lower index (first maximum).
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// ---- shared-memory barriers and bulk tensor copies ---------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^31 clock ticks (about a second) and returns false, so that a
// lost copy can never hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > (1ll << 31)) return false;
    }
    return true;
}
// 2-D tiled bulk copy global -> shared of one box of the tensor map, completing on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// The same copy with an L2 eviction policy (weights are read once per token: evict_first keeps them from
// displacing the small data every operator re-reads: activations, group constants, the KV cache).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(pol) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- programmatic dependent launch ----------------------------------------------------------------
// wait: blocks until the kernels this launch depends on have completed and their writes are
// visible (no-op for a plain launch).  launch_dependents: lets the next kernel's CTAs be
// scheduled as soon as this grid's CTAs have all passed this point and SM resources free up.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- warp-level tensor op: D(16x8,f32) += A(16x16,f16) * B(16x8,f16) ------------------------------
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ double shfl_xor_double(double v, int mask) {
    int lo = __double2loint(v), hi = __double2hiint(v);
    lo = __shfl_xor_sync(0xffffffffu, lo, mask);
    hi = __shfl_xor_sync(0xffffffffu, hi, mask);
    return __hiloint2double(hi, lo);
}

// erf-GeLU of an fp16 value (Inference.cu:271-279).
__device__ __forceinline__ __half gelu_h(__half h) {
    float v = __half2float(h);
    float y = 0.5f * v * (1.0f + erff(v * 0.70710678f));
    return __float2half_rn(y);
}

#endif  // __CUDACC__

}  // namespace qw3
