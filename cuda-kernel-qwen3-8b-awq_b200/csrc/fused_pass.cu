// Fused token pass (sm_100a): one persistent cooperative kernel per token and GPU, with the operators of a layer
// paired so that only two grid-wide reductions per layer remain.
//
// The reference runs a token through a layer as 12 launches and 68 copies (runOneLayer, Inference.cu:1029-1230).  At
// batch 1 a layer's 84 MB of packed weights take 12.8 us of HBM time, so what sets the pace is how often the whole
// grid has to agree on a vector.  Here every head gets a group of `gs` CTAs:
//   group of head h:  RMSNorm -> its K-slice of Wqkv for q_h, k_h, v_h -> (group exchange) -> RoPE, KV append,
//                     attention over its share of the positions -> (group exchange) -> Wo restricted to the 128
//                     context inputs of head h, for its share of the outputs
//   grid:             ordered sum of the per-head partial outputs + residual (every CTA owns `rs` hidden elements),
//                     then the new hidden state is gathered by everybody
//   every CTA:        RMSNorm -> its n1 outputs of W1 -> GeLU -> W2 restricted to those n1 inputs, all outputs
//   grid:             ordered sum + residual, gather
// Everything that crosses CTAs travels as (payload, tag) in one aligned 64-bit word which the reader polls: the tag
// names generation, position and phase, so nothing is ever cleared and a CUDA graph replays unchanged.  Sums run in a
// fixed order: results are bitwise repeatable.  With the matrices row-split over several GPUs (one process per GPU)
// the same words are stored into every GPU's copy of the exchange buffers over NVLink and polled locally.
//
// Weights: every matrix is rewritten at load time (fused_plan.h) into per-(CTA, warp) byte streams in consumption
// order, the 16 warp streams of a CTA interleaved in units.  A ring of FP_SLOTS slots per CTA holds the units in flight:
// one 1-D bulk copy (L2 evict-first) per unit; a warp counts itself off a unit once its last loads of it are issued and
// the sixteenth warp refills the slot, across operator boundaries, since weights never depend on activations.
// On one GPU the CTAs of a head can form a thread-block cluster (FusedParams::cluster): the two exchanges inside the
// group then go through distributed shared memory instead of global memory.
// Inner loop: the integer tensor-core path.  One 16-byte shared-memory load per lane yields four words; `w & 0x0f0f0f0f`
// and `w & 0xf0f0f0f0` of two words ARE the u8 A fragment of mma.sync.m16n8k32 (u8 x s8 -> s32): the low nibbles of a
// word are four weights of row g, the high nibbles four weights of row g + 8 times 16.  The activations of the
// operator are brought to fixed point once per CTA, X_j = rint(x_j * 2^sh) with |X_j| < 2^22 (fp16 values within 2^11
// of the largest are exact, the others are off by at most 2^-23 of the largest), and split into three signed base-256
// digits which sit in columns 0, 1, 2 of the B fragment.  So the tensor core accumulates sum_j q_ij X_j exactly, in
// three s32 columns, and the epilogue applies  y_i = scale_i * (2^-sh * (65536 D_i0 + 256 D_i1 + D_i2) - zp_i * sum_j x_j):
// two integer instructions per eight weights and one MMA per sixteen (the fp16 form of the same loop, nibbles as
// subnormal fp16 into m16n8k16, needed five and two and ran half as fast: mma.sync issues at the same rate for both
// shapes on this part).  This is algebraically the reference's (q - zp) * scale product (Inference.cu:102-104) without
// its two fp16 roundings per weight; the bit-exact form stays in qw3_dequant_w4, in the stand-alone GEMV and in the
// tensor-core GEMM, and the tests hold this kernel to the logits tolerance.
// The unembedding's groups depend on the input index; there the scale is folded into the activations per block of
// 128 outputs (x'_j = scale_g(b,j) * x_j) and the same loop runs.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "fused_pass.h"

namespace qw3 {

constexpr int FP_NT = F_NW * 32;          // threads per CTA
#ifndef QW3_FP_SLOTS
#define QW3_FP_SLOTS 3
#endif
constexpr int FP_SLOTS = QW3_FP_SLOTS;    // ring units in flight
constexpr int FP_MAX_H = 4096;            // largest hidden size (activation vectors kept in shared memory)
constexpr int FP_OBUF = 4608;             // floats: GEMV outputs / partial-sum staging / 32 attention states of 132
constexpr int FP_MAX_SEG = 4 * 64 + 24;   // weight segments of one pass (4 per layer + unembedding rounds)
constexpr int FP_MAX_N1 = 512;            // largest number of W1 outputs per CTA
constexpr int FP_MAX_RS = 256;            // largest number of hidden elements a CTA owns
constexpr int FP_ATT_STRIDE = 132;
constexpr int FP_MAX_GROUPS = 128;        // largest number of scale / zero-point entries of a layer matrix
constexpr int FP_QKV = 384;               // q, k, v of one head

constexpr size_t FP_OFF_OBUF = (size_t)FP_SLOTS * F_NW * F_UNIT;
constexpr size_t FP_OFF_HV = FP_OFF_OBUF + (size_t)FP_OBUF * 4;
constexpr size_t FP_OFF_XS = FP_OFF_HV + (size_t)FP_MAX_H * 2;
constexpr size_t FP_OFF_SEG = FP_OFF_XS + (size_t)FP_MAX_H * 3;   // three digit planes of FP_MAX_H bytes
constexpr size_t FP_OFF_LSZ = FP_OFF_SEG + (size_t)FP_MAX_SEG * 16;          // [2][4][FP_MAX_GROUPS] (scale, zero point) as floats
constexpr size_t FP_OFF_MISC = FP_OFF_LSZ + (size_t)2 * 4 * FP_MAX_GROUPS * 8;
constexpr size_t FP_MISC_BYTES = 8192;
constexpr int FP_CL_MAX = 4;              // largest head group that exchanges through distributed shared memory (one thread-block cluster)
constexpr size_t FP_OFF_CL = FP_OFF_MISC + FP_MISC_BYTES;                    // xq_in [FP_CL_MAX][FP_QKV], xa_in [FP_CL_MAX][FP_ATT_STRIDE] floats, 2 barriers
constexpr size_t FP_CL_BYTES = (size_t)FP_CL_MAX * (FP_QKV + FP_ATT_STRIDE) * 4 + 64;
constexpr size_t FP_SMEM_BYTES = FP_OFF_CL + FP_CL_BYTES;

struct FLayerDesc {
    const uint8_t* w[4];        // repacked Wqkv, Wo, W1, W2 of this rank
    const __half* scale[4];
    const __half* zp[4];
    const __half* gamma;
    __half* kc;
    __half* vc;
};

// Descriptor plus the scale / zero-point entries of the four matrices, one flat block per layer (built on the device
// at load time), so that a pass fetches it with single-level loads.
struct FLayerConst {
    FLayerDesc d;
    uint32_t sz[4][FP_MAX_GROUPS];   // (scale, zero point) as two halves
};

struct FusedParams {
    const FLayerConst* layers;
    int n_layers;
    FusedGeom g;
    FGemvPlan plan[F_NOPS];
    int n_alloc[F_NOPS];          // scale / zero-point entries of each matrix kind
    int n_rounds;                 // unembedding rounds (0: this pass does not sample)
    int hpr_shift, rs_shift;      // log2 of H / n_ranks and of rs when those are powers of two, else -1
    float eps;
    int attn_split_min;
    // embedding (first stage) and unembedding (last stage)
    const uint8_t* emb_packed; const __half* emb_scale; const __half* emb_zp; int emb_n_alloc;
    const uint8_t* un_w; const __half* un_scale; const __half* un_zp;
    const __half* gamma_final;
    __half* logits16; float* logits32;
    int first_stage;
    // sequence state
    __half* hidden;               // residual stream between passes (plain)
    const int* d_pos; const int* d_token; const int* d_skip; const int* d_prompt; const int* d_gen;
    int decode;
    int cluster;                  // 1: the gs CTAs of a head are one thread-block cluster and exchange through distributed shared memory
    int dry;                      // 1: the launch only proves that the configuration can be launched (every CTA returns after the cluster barrier)
    const __half* cos_t; const __half* sin_t;
    long long max_pos;
    int* d_token_out;
    // exchange buffers of tagged words; index [r] is rank r's copy (a peer mapping when r != rank)
    unsigned long long* xq;                    // [n_act][384]                 q/k/v partial sums (group-local)
    unsigned long long* xa;                    // [n_act][132]                 attention states (group-local)
    unsigned long long* xo[QW3_MAX_STAGES];    // [heads * gs][H / gs]         Wo partial sums per (head, output share)
    unsigned long long* x2[QW3_MAX_STAGES];    // [n_ranks * n_mlp][H]         W2 partial sums per contributor
    unsigned long long* hid[QW3_MAX_STAGES];   // [2][H / 2]                   gathered hidden state, two buffers
    unsigned long long* xarg[QW3_MAX_STAGES];  // [n_ranks * grid][2]          arg-max candidates
    int* err;
    unsigned long long* trace;    // tracing builds (-DQW3_TRACE): [grid][n_layers][16] global-timer stamps of thread 0
};

#ifdef QW3_TRACE
#define FP_STAMP(li, k)                                                                              \
    do {                                                                                             \
        if (threadIdx.x == 0 && p.trace != nullptr) {                                                \
            unsigned long long t__;                                                                  \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t__));                                   \
            p.trace[((size_t)blockIdx.x * p.n_layers + (li)) * 16 + (k)] = t__;                       \
        }                                                                                            \
    } while (0)
// Cycle stamps of the warps of CTA 0 inside the GEMV of operator `op` (tail of the trace buffer: [op][warp][8]).
#define FP_WSTAMP(op, k)                                                                                   \
    do {                                                                                                   \
        extern __shared__ __align__(1024) uint8_t smem_w__[];                                              \
        unsigned long long* tr__ = *reinterpret_cast<unsigned long long**>(smem_w__ + FP_OFF_MISC + 3680); \
        if (tr__ != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0)                                 \
            tr__[(op) * 128 + (threadIdx.x >> 5) * 8 + (k)] = (unsigned long long)clock64();               \
    } while (0)
// Warp 0 of CTA 0: cycle stamps before / after the wait for unit `u` of operator `op` ([op][32][2] after the warp stamps).
#define FP_USTAMP(op, u, k)                                                                                \
    do {                                                                                                   \
        extern __shared__ __align__(1024) uint8_t smem_w__[];                                              \
        unsigned long long* tr__ = *reinterpret_cast<unsigned long long**>(smem_w__ + FP_OFF_MISC + 3680); \
        if (tr__ != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && (u) < 32)                            \
            tr__[640 + ((op) * 32 + (u)) * 2 + (k)] = (unsigned long long)clock64();                       \
    } while (0)
#else
#define FP_STAMP(li, k) do { } while (0)
#define FP_WSTAMP(op, k) do { } while (0)
#define FP_USTAMP(op, u, k) do { } while (0)
#endif

// ---- tagged words ------------------------------------------------------------------------------------------------
template <bool SYS>
__device__ __forceinline__ unsigned long long ldt(const unsigned long long* p) {
    unsigned long long a;
    if (SYS) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}
template <bool SYS>
__device__ __forceinline__ void ldt2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    if (SYS) asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// Four adjacent words by one 32-byte load (the address is 32-byte aligned).  Every word is still checked by its own tag:
// nothing here relies on the four arriving together.
template <bool SYS>
__device__ __forceinline__ void ldt4(const unsigned long long* p, unsigned long long (&w)[4]) {
    if (SYS) asm volatile("ld.relaxed.sys.global.v4.b64 {%0, %1, %2, %3}, [%4];" : "=l"(w[0]), "=l"(w[1]), "=l"(w[2]), "=l"(w[3]) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.v4.b64 {%0, %1, %2, %3}, [%4];" : "=l"(w[0]), "=l"(w[1]), "=l"(w[2]), "=l"(w[3]) : "l"(p) : "memory");
}
template <bool SYS>
__device__ __forceinline__ void stt(unsigned long long* p, unsigned long long a) {
    if (SYS) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
    else asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
template <bool SYS>
__device__ __forceinline__ void stt2(unsigned long long* p, unsigned long long a, unsigned long long b) {
    if (SYS) asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
    else asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ unsigned long long tagged(uint32_t payload, uint32_t tag) {
    return ((unsigned long long)tag << 32) | payload;
}
__device__ __forceinline__ unsigned long long tagged_f(float v, uint32_t tag) { return tagged(__float_as_uint(v), tag); }
__device__ __forceinline__ bool has_tag(unsigned long long w, uint32_t tag) { return (uint32_t)(w >> 32) == tag; }
__device__ __forceinline__ float payload_f(unsigned long long w) { return __uint_as_float((uint32_t)w); }

constexpr long long FP_WAIT_LOCAL = 1ll << 31;   // about a second
constexpr long long FP_WAIT_PEER = 1ll << 33;    // words another GPU writes

// ---- shared-memory views and per-pass constants ---------------------------------------------------------------------
struct FCtx {
    uint8_t* ring;
    float* obuf;
    __half* hv;
    uint8_t* xd;        // [3][FP_MAX_H] digits of the fixed-point activations of the operator about to run (plane c = digit c, most significant first)
    float* xinv;        // 2^-sh of those activations
    float* xq_in;       // [gs][FP_QKV] cluster exchange: slot r is written by CTA r of the head group (into every member's copy)
    float* xa_in;       // [gs][FP_ATT_STRIDE]
    uint32_t cl_bars;   // shared address of the two barriers of the cluster exchange (xq, xa)
    int4* seg;          // {base lo, base hi, warp_bytes, unit_bytes} per weight segment of this CTA
    float2* lsz;        // [2][4][FP_MAX_GROUPS] (scale, zero point) of the layer's four matrices, two layers (current / next)
    FLayerDesc* ldesc;  // [2] descriptor of the current / next layer
    __half* qkv_s;      // [384] q, k, v of this CTA's head (after RoPE)
    __half* hmine;      // [rs] this CTA's part of the residual stream
    __half* rope_cs;    // [128] cos | sin of this position
    float* wsum;        // [64]
    float* bsm;         // [2][2 * F_NW] scratch rows of block_sum_max
    float* gsm;         // [2][3 * F_NW] scratch rows of gather_norm (with dsum [2][F_NW])
    double* dsum;       // [16]
    uint32_t* un_sz;    // [<= 64] scale | zp pairs of the unembedding groups in use
    float* argv;        // [16]
    int* argi;          // [16]
    int* s_dead;
    int* err;           // device error word of the launch
    const FGemvPlan* plans;   // [F_NOPS] the operator plans, copied to shared memory for the out-of-line GEMV
    const int4* wplan;        // [F_NOPS][F_NW] per operator and warp: {byte offset of its k-share in a digit plane, float offset of its sums in obuf, units per block, groups per unit}
    int* ring_cnt;      // [FP_SLOTS] warps that have consumed their piece of the unit in the slot
    int* ring_issued;   // units requested so far (only the issuing thread of the moment writes it)
    uint32_t bars;      // shared address of the ring barriers [FP_SLOTS]
    uint32_t zero_addr; // shared address of 32 zero bytes
    uint32_t tagbase;
    int pos;
    int n_seg;
};

__device__ __forceinline__ void fail(const FCtx& cx, int code) {
    atomicCAS(cx.err, 0, code);
    *cx.s_dead = 1;
}

// Up to NB words polled together (all loads in flight at once) until every one carries `tag`; bounded.  A word that
// has arrived is not loaded again: re-reading the arrived ones in every round was measured to cost 2-3 us per
// grid-wide reduction (the rounds compete in L2 with the stores they wait for).
template <bool SYS, int NB, typename AddrFn>
__device__ __forceinline__ void poll_batch(const FusedParams& p, const FCtx& cx, const int n_valid, AddrFn addr, const uint32_t tag,
                                           const int code, unsigned long long (&w)[NB]) {
    const long long t_begin = clock64();
    bool have[NB];
#pragma unroll
    for (int e = 0; e < NB; ++e) have[e] = e >= n_valid;
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int e = 0; e < NB; ++e) {
            if (!have[e]) {
                w[e] = ldt<SYS>(addr(e));
                have[e] = has_tag(w[e], tag);
            }
            ok = ok && have[e];
        }
        if (ok || *cx.s_dead != 0) break;
        if (clock64() - t_begin > (SYS ? FP_WAIT_PEER : FP_WAIT_LOCAL)) {
            fail(cx, code);
            break;
        }
    }
}

// The same for PAIRS of adjacent words (one 16-byte load each): addr(e) is the first word of pair e, 16-byte aligned.
template <bool SYS, int NB, typename AddrFn>
__device__ __forceinline__ void poll_pairs(const FusedParams& p, const FCtx& cx, const int n_valid, AddrFn addr, const uint32_t tag,
                                           const int code, unsigned long long (&w)[NB][2]) {
    const long long t_begin = clock64();
    bool have[NB];
#pragma unroll
    for (int e = 0; e < NB; ++e) have[e] = e >= n_valid;
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int e = 0; e < NB; ++e) {
            if (!have[e]) {
                ldt2<SYS>(addr(e), w[e][0], w[e][1]);
                have[e] = has_tag(w[e][0], tag) && has_tag(w[e][1], tag);
            }
            ok = ok && have[e];
        }
        if (ok || *cx.s_dead != 0) break;
        if (clock64() - t_begin > (SYS ? FP_WAIT_PEER : FP_WAIT_LOCAL)) {
            fail(cx, code);
            break;
        }
    }
}

// The same for groups of FOUR adjacent words (one 32-byte load each): addr(e) is 32-byte aligned.
template <bool SYS, int NB, typename AddrFn>
__device__ __forceinline__ void poll_quads(const FusedParams& p, const FCtx& cx, const int n_valid, AddrFn addr, const uint32_t tag,
                                           const int code, unsigned long long (&w)[NB][4]) {
    const long long t_begin = clock64();
    bool have[NB];
#pragma unroll
    for (int e = 0; e < NB; ++e) have[e] = e >= n_valid;
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int e = 0; e < NB; ++e) {
            if (!have[e]) {
                ldt4<SYS>(addr(e), w[e]);
                have[e] = has_tag(w[e][0], tag) && has_tag(w[e][1], tag) && has_tag(w[e][2], tag) && has_tag(w[e][3], tag);
            }
            ok = ok && have[e];
        }
        if (ok || *cx.s_dead != 0) break;
        if (clock64() - t_begin > (SYS ? FP_WAIT_PEER : FP_WAIT_LOCAL)) {
            fail(cx, code);
            break;
        }
    }
}

// ---- weight ring -----------------------------------------------------------------------------------------------------
// The CTA's weight stream is a sequence of units; a unit holds one piece of up to F_UNIT bytes for each of the 16
// warps, contiguous in global memory ([warp][piece]), and is fetched by ONE bulk copy (32 KB): bulk copies cost a
// fixed ~140 ns each on this part whatever their size, so one copy per warp and piece would cap an SM at ~15 GB/s.
// FP_SLOTS units are in flight.  Every warp consumes its piece of a unit, then counts itself off on the slot; the
// last warp to do so issues the copy of the unit FP_SLOTS places ahead into that slot.  All warps walk the same unit
// sequence, so each keeps the cursor in its own registers and no shared producer state exists.
struct WarpRing {
    int uc;        // units consumed by this warp so far
    int pseg, pu;  // unit FP_SLOTS places ahead of uc: segment and unit within it (pseg == n_seg: past the end)
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}

// Moves the cursor to the next unit this CTA has (segments it takes no part in have no bytes).  Returns false past the end.
__device__ __forceinline__ bool ring_cursor_valid(WarpRing& r, const FCtx& cx) {
    while (r.pseg < cx.n_seg) {
        const int4 sg = cx.seg[r.pseg];
        if (r.pu * sg.w < sg.z) return true;
        ++r.pseg;
        r.pu = 0;
    }
    return false;
}
// Issues the bulk copy of the unit under the cursor into `slot` (one thread calls this) and advances nothing.
__device__ __forceinline__ void ring_issue(const WarpRing& r, const FCtx& cx, const int slot) {
    const int4 sg = cx.seg[r.pseg];
    const uint8_t* base = reinterpret_cast<const uint8_t*>(((unsigned long long)(uint32_t)sg.y << 32) | (uint32_t)sg.x);
    const int piece = sg.w;
    const uint32_t bar = cx.bars + 8 * slot;
    // The slot was read with ordinary loads that have all completed (every warp counted itself off with a release
    // operation after issuing its last loads of the piece), so the bulk write cannot overtake them; no proxy fence is
    // needed for this read-then-overwrite order, and one here would wait for the copies still in flight into the
    // other slots (measured: no difference in results, slower).
    *cx.ring_issued += 1;
    mbar_expect_tx(bar, F_NW * piece);
    bulk_load(smem_u32(cx.ring) + slot * (F_NW * F_UNIT), base + (size_t)r.pu * (F_NW * piece), F_NW * piece, bar, l2_policy_evict_first());
}

// Shared address of this warp's piece (of `piece` bytes) of the unit it consumes next, once the unit has landed.
__device__ __forceinline__ uint32_t ring_wait(const WarpRing& r, const FCtx& cx, const int piece) {
    const int warp = threadIdx.x >> 5, slot = r.uc % FP_SLOTS;
    uint32_t addr = smem_u32(cx.ring) + slot * (F_NW * F_UNIT) + warp * piece;
#ifndef QW3_FP_NOLOAD
    // One lane polls the barrier (barrier operations of a CTA are served one at a time: 512 threads polling cost more
    // than the piece's arithmetic); the warp barrier hands the observation, and the memory order it implies, to the others.
    if ((threadIdx.x & 31) == 0) {
        if (*cx.s_dead == 0 && !mbar_wait(cx.bars + 8 * slot, (r.uc / FP_SLOTS) & 1)) {
            if ((threadIdx.x & 31) == 0) fail(cx, 0x10000 | (r.uc & 0xffff));   // a weight unit never arrived
        }
    }
    __syncwarp();
#endif
    asm volatile("" : "+r"(addr));   // loads from the unit use this value: none is scheduled before the wait
    return addr;
}
// This warp is done with its piece of unit uc: the last of the 16 warps refills the slot.  After a wait has given up
// nothing more is requested.
__device__ __forceinline__ void ring_release(WarpRing& r, const FCtx& cx) {
    __syncwarp();
    const int slot = r.uc % FP_SLOTS;
    const bool more = ring_cursor_valid(r, cx);
#ifndef QW3_FP_NOLOAD
    if ((threadIdx.x & 31) == 0) {
        uint32_t old;
        asm volatile("atom.release.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(cx.ring_cnt + slot)) : "memory");
        if (old == F_NW - 1) {
            cx.ring_cnt[slot] = 0;
            if (more && *cx.s_dead == 0) ring_issue(r, cx, slot);
        }
    }
#endif
    if (more) ++r.pu;
    ++r.uc;
}

// Shared-memory loads of the weight stream and of the B fragments.  Volatile, so that the compiler keeps them between
// the wait for their unit and the count that releases it (both volatile); the MMAs are free to move.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Two words of a lane = one A fragment: low nibbles -> rows g, high nibbles -> rows g + 8 (sixteen-fold).
__device__ __forceinline__ void mma_pair(int (&d)[4], uint32_t wa, uint32_t wb, uint32_t b0, uint32_t b1) {
#ifdef QW3_FP_NOCOMPUTE
    d[0] += (int)(wa & wb & b0 & b1);   // timing experiment: the weights only stream through (results are meaningless)
    return;
#endif
    mma_u8s8(d, wa & 0x0f0f0f0fu, wa & 0xf0f0f0f0u, wb & 0x0f0f0f0fu, wb & 0xf0f0f0f0u, b0, b1);
}

// ---- fixed-point activations ------------------------------------------------------------------------------------------------
// bound >= max |x_j|  ->  up = 2^sh with |x_j| * 2^sh < 2^22, inv = 2^-sh.
struct XScale { float up, inv; };
__device__ __forceinline__ XScale xscale_for(float bound) {
    int e = (int)((__float_as_uint(bound) >> 23) & 0xffu) - 126;   // bound < 2^e (normal floats; tiny bounds are clamped below)
    int sh = 22 - e;
    sh = max(-100, min(100, sh));
    XScale r;
    r.up = __uint_as_float((uint32_t)(sh + 127) << 23);
    r.inv = __uint_as_float((uint32_t)(127 - sh) << 23);
    return r;
}
__device__ __forceinline__ int xfix(__half x, const XScale& q) {
    const int X = __float2int_rn(__half2float(x) * q.up);
    return max(-(1 << 22), min(1 << 22, X));   // a non-finite activation must not leave the digit range
}
// X = 65536 h + 256 m + l with m, l in [-128, 127]; byte k of `pack` receives the digit.
__device__ __forceinline__ void xdigits(int X, int k, uint32_t& ph, uint32_t& pm, uint32_t& pl) {
    const int l = ((X + 128) & 255) - 128;
    X = (X - l) >> 8;
    const int m = ((X + 128) & 255) - 128;
    const int h = (X - m) >> 8;
    ph |= (uint32_t)(h & 255) << (8 * k);
    pm |= (uint32_t)(m & 255) << (8 * k);
    pl |= (uint32_t)(l & 255) << (8 * k);
}

// This warp's stream of one operator: nb blocks of TB tiles, each over nq groups of 64 inputs (+ a half group of 32 when
// rem == 2).  The stream comes in ring units of whole groups (gu of them; a block with a half group is one unit), so
// that one barrier wait is followed by straight-line code: every load of the unit can be issued ahead of its MMAs.
// xd_addr: shared address of the most significant digit plane at the warp's k-share.  dst[(block * TB + i) * 16 + row]
// receives sum_j q[row][j] * x[j] of tile i of the block.  Tiles of a block are issued one after another per group, so
// TB (2 * TB for narrow blocks) independent MMA chains are in flight.
template <int TB>
__device__ __forceinline__ void gemv_core(const FCtx& cx, WarpRing& ring, const FGemvPlan& pl, const uint32_t xd_addr, float* dst, const int op,
                                          const int upb, const int ng) {   // units per block, full groups per unit
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nq = pl.nq, rem = pl.rem;
    constexpr int NA = TB <= 3 ? 2 : 1;   // accumulators per tile: the two MMAs of a group never wait for each other (six chains at
                                          // TB = 3: 2.5 % in tokens/s over one accumulator; at TB = 4 the second set costs registers: slower)
    // B fragment: column g of the MMA is digit plane g (columns 3-7 are zero); lane t holds 16 consecutive inputs of a group
    const bool col = g < 3;
    const uint32_t bbase = xd_addr + g * FP_MAX_H + t * 16, bhalf = xd_addr + g * FP_MAX_H + nq * 64 + t * 8;
    const float inv = *cx.xinv;
    uint32_t next_base = ring_wait(ring, cx, pl.unit_bytes);
    FP_WSTAMP(op, 1);
    for (int b = 0; b < pl.nb; ++b) {
        int acc[TB][NA][4];
#pragma unroll
        for (int i = 0; i < TB; ++i)
#pragma unroll
            for (int h = 0; h < NA; ++h)
#pragma unroll
                for (int d = 0; d < 4; ++d) acc[i][h][d] = 0;
        for (int uu = 0; uu < upb; ++uu) {
            const uint32_t ubase = next_base;
            uint32_t a = ubase + lane * 16;
            const uint32_t xq = bbase + uu * ng * 64;
            for (int gq = 0; gq < ng; ++gq) {
                const uint4 bv = lds128(col ? xq + gq * 64 : cx.zero_addr);
                uint4 w[TB];
#pragma unroll
                for (int i = 0; i < TB; ++i) w[i] = lds128(a + i * 512);
                a += TB * 512;
                if (rem != 2 && gq + 1 == ng) {   // the unit's last loads are issued
                    if (b == 0 && uu == 0) FP_WSTAMP(op, 2);
                    ring_release(ring, cx);
                    if (b == 0 && uu == 0) FP_WSTAMP(op, 3);
                    if (uu + 1 < upb || b + 1 < pl.nb) next_base = ring_wait(ring, cx, pl.unit_bytes);
                    if (b == 0 && uu == 0) FP_WSTAMP(op, 5);
                }
#pragma unroll
                for (int i = 0; i < TB; ++i) mma_pair(acc[i][0], w[i].x, w[i].y, bv.x, bv.y);
#pragma unroll
                for (int i = 0; i < TB; ++i) mma_pair(acc[i][NA - 1], w[i].z, w[i].w, bv.z, bv.w);
            }
            if (rem == 2) {
                const uint2 bv = lds64(col ? bhalf : cx.zero_addr);
                const uint32_t h = ubase + nq * TB * 512 + lane * 8;
                uint2 w[TB];
#pragma unroll
                for (int i = 0; i < TB; ++i) w[i] = lds64(h + i * 256);
                ring_release(ring, cx);
                if (uu + 1 < upb || b + 1 < pl.nb) next_base = ring_wait(ring, cx, pl.unit_bytes);
#pragma unroll
                for (int i = 0; i < TB; ++i) mma_pair(acc[i][0], w[i].x, w[i].y, bv.x, bv.y);
            }
        }
        // D: lane t = 0 holds columns 0, 1 (digits 65536, 256) of rows g (d0, d1) and g + 8 (d2, d3), lane t = 1 column 2 (d0, d2)
        if (b + 1 == pl.nb) FP_WSTAMP(op, 6);
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            int d[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) d[k] = NA == 2 ? acc[i][0][k] + acc[i][NA - 1][k] : acc[i][0][k];
            const float lo_g = __shfl_down_sync(0xffffffffu, (float)d[0], 1), lo_g8 = __shfl_down_sync(0xffffffffu, (float)d[2], 1);
            if (t == 0) {
                dst[(b * TB + i) * 16 + g] = fmaf(65536.0f, (float)d[0], fmaf(256.0f, (float)d[1], lo_g)) * inv;
                dst[(b * TB + i) * 16 + g + 8] = fmaf(65536.0f, (float)d[2], fmaf(256.0f, (float)d[3], lo_g8)) * (inv * 0.0625f);
            }
        }
    }
}

__device__ __forceinline__ FCtx carve_ctx(uint8_t* smem);

// Runs this warp's share of operator `op`: warp (a, bk) of the plan; sums land in obuf[bk][tile * 16 + row].
// ONE out-of-line copy serves the four operators of a layer and the unembedding (inlined at every call site the
// loop was in the kernel twenty times, and a pass spent a sixth of its issue slots waiting for instructions).  The
// function takes and returns the ring cursor in registers and finds everything else in shared memory, so nothing of
// it lives in local memory.
__device__ __noinline__ int3 gemv_entry(const int uc, const int pseg, const int pu, const int op, const uint32_t x_cta_addr) {
    extern __shared__ __align__(1024) uint8_t smem[];
    FP_WSTAMP(op, 0);
    const FCtx cx = carve_ctx(smem);
    WarpRing ring;
    ring.uc = uc; ring.pseg = pseg; ring.pu = pu;
    const FGemvPlan& pl = cx.plans[op];
    const int4 wp = cx.wplan[op * F_NW + (threadIdx.x >> 5)];
    const uint32_t xs_addr = x_cta_addr + wp.x;
    float* dst = cx.obuf + wp.y;
    switch (pl.tb) {
        case 1: gemv_core<1>(cx, ring, pl, xs_addr, dst, op, wp.z, wp.w); break;
        case 2: gemv_core<2>(cx, ring, pl, xs_addr, dst, op, wp.z, wp.w); break;
        case 3: gemv_core<3>(cx, ring, pl, xs_addr, dst, op, wp.z, wp.w); break;
        default: gemv_core<4>(cx, ring, pl, xs_addr, dst, op, wp.z, wp.w); break;
    }
    FP_WSTAMP(op, 4);
    return make_int3(ring.uc, ring.pseg, ring.pu);
}
// x_cta: the first input of the CTA within the digit planes (cx.xd + offset)
__device__ __forceinline__ void run_gemv(WarpRing& ring, const int op, const uint8_t* x_cta) {
    const int3 r = gemv_entry(ring.uc, ring.pseg, ring.pu, op, smem_u32(x_cta));
    ring.uc = r.x; ring.pseg = r.y; ring.pu = r.z;
}
__device__ __forceinline__ float sum_k_shares(const FCtx& cx, const FGemvPlan& pl, int i) {
    float s = 0.0f;
    for (int bk = 0; bk < pl.wk; ++bk) s += cx.obuf[bk * (pl.n_mt * 16) + i];
    return s;
}

// Scale and zero point of output `o` of a matrix whose groups do not depend on the input index.  The table holds one
// entry per block of 128 outputs: entry b = (scale, zero point) of group ((b mod (in_dim / 128)) mod entries), i.e.
// dequantAwqKernel's c / 128 with the wrapped index (Inference.cu:90), resolved once at load time (fused_consts_kernel).
__device__ __forceinline__ void group_consts(const float2* table, long long o, float& s, float& z) {
    const float2 v = table[o >> 7];
    s = v.x;
    z = v.y;
}

// Scale / zero-point tables and descriptor of a layer: requested from global memory a whole layer before they are
// needed (the values sit in registers meanwhile), so that no epilogue waits for a global load.
struct LayerPrefetch {
    uint32_t sz;                 // threads 0 .. 4 * FP_MAX_GROUPS - 1: (scale, zp) bits of entry tid % FP_MAX_GROUPS of matrix tid / FP_MAX_GROUPS
    unsigned long long word;     // threads 0 .. sizeof(FLayerDesc) / 8 - 1: one word of the descriptor
};
__device__ __forceinline__ void layer_request(const FusedParams& p, int li, LayerPrefetch& lp) {
    const int tid = threadIdx.x;
    lp.sz = 0u;
    lp.word = 0ull;
    if (li >= p.n_layers) return;
    const FLayerConst& L = p.layers[li];
    static_assert(4 * FP_MAX_GROUPS == FP_NT && sizeof(FLayerDesc) % 8 == 0 && sizeof(FLayerDesc) / 8 <= FP_NT, "one entry per thread");
    lp.sz = __ldg(&L.sz[0][0] + tid);
    if (tid < (int)(sizeof(FLayerDesc) / 8)) lp.word = __ldg(reinterpret_cast<const unsigned long long*>(&L.d) + tid);
}
__device__ __forceinline__ void layer_commit(const FCtx& cx, int buf, const LayerPrefetch& lp) {
    const int tid = threadIdx.x;
    cx.lsz[buf * 4 * FP_MAX_GROUPS + tid] = make_float2(__half2float(__ushort_as_half((unsigned short)(lp.sz & 0xffffu))),
                                                        __half2float(__ushort_as_half((unsigned short)(lp.sz >> 16))));
    if (tid < (int)(sizeof(FLayerDesc) / 8)) reinterpret_cast<unsigned long long*>(cx.ldesc + buf)[tid] = lp.word;
}

__device__ __forceinline__ float block_sum_f(const FCtx& cx, float v) {   // all threads call; fixed order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    __syncthreads();
    if (lane == 0) cx.wsum[warp] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < F_NW; ++w) s += cx.wsum[w];
    return s;
}

// Sum of v and maximum of a (a >= 0) over the CTA; all threads call.  `which` (0 / 1) names one of two scratch rows: the
// two calls of a layer alternate, and a row's readers of the layer before are many barriers away, so ONE barrier does.
__device__ __forceinline__ void block_sum_max(const FCtx& cx, const int which, float v, float a, float& sum, float& amax) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, m);
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, m));
    }
    float* row = cx.bsm + which * 2 * F_NW;
    if (lane == 0) {
        row[warp] = v;
        row[F_NW + warp] = a;
    }
    __syncthreads();
    sum = 0.0f;
    amax = 0.0f;
#pragma unroll
    for (int w = 0; w < F_NW; ++w) {
        sum += row[w];
        amax = fmaxf(amax, row[F_NW + w]);
    }
}
// A short activation vector (one element per thread, `n` of them) to the digit planes; a barrier must follow.
__device__ __forceinline__ void quantise_own(const FCtx& cx, const __half v, const int n, const float amax) {
    const int tid = threadIdx.x;
    const XScale xq = xscale_for(amax);
    if (tid < n) {
        uint32_t ph = 0u, pm = 0u, pl = 0u;
        xdigits(xfix(v, xq), 0, ph, pm, pl);
        cx.xd[tid] = (uint8_t)ph;
        cx.xd[FP_MAX_H + tid] = (uint8_t)pm;
        cx.xd[2 * FP_MAX_H + tid] = (uint8_t)pl;
    }
    if (tid == 0) *cx.xinv = xq.inv;
}

// ---- gather of the hidden state + RMSNorm (rmsNormKernel, Inference.cu:111-145) --------------------------------------
// Polls the H/2 tagged words of `hid` and normalises with `gamma`.  QUANT: the result goes to the digit planes in fixed
// point (the B operand of the operator that follows) and x_full / x_slice are the sums of those fixed-point values:
// x_full over the whole vector, x_slice over [slice * hs, (slice + 1) * hs) (hs a multiple of 128).  Otherwise the fp16
// result goes to `out` (shared memory) and `bound` receives an upper bound of its absolute values.
template <bool SYS, bool QUANT>
__device__ __forceinline__ void gather_norm(const FusedParams& p, const FCtx& cx, const unsigned long long* hid, const uint32_t tag,
                                            const __half* gamma, __half* out, const int slice, const int hs, float& x_full,
                                            float& x_slice, float& bound, const int which) {   // which (0 / 1): scratch row; successive calls alternate
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* const row = cx.gsm + which * 3 * F_NW;   // [2 * F_NW] sums, [F_NW] maxima
    double* const drow = cx.dsum + which * F_NW;
    const int H = p.g.H, nch = H >> 2;   // chunks of two words = four halves
    unsigned long long w[2][2] = {{0ull, 0ull}, {0ull, 0ull}};
    uint2 gm[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int ch = tid + e * FP_NT;
        if (ch < nch) gm[e] = __ldg(reinterpret_cast<const uint2*>(gamma) + ch);
    }
    const long long t_begin = clock64();
    bool have[2] = {tid >= nch, tid + FP_NT >= nch};
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (!have[e]) {
                ldt2<SYS>(hid + 2 * (tid + e * FP_NT), w[e][0], w[e][1]);
                have[e] = has_tag(w[e][0], tag) && has_tag(w[e][1], tag);
            }
            ok = ok && have[e];
        }
        if (ok || *cx.s_dead != 0) break;
        if (clock64() - t_begin > (SYS ? FP_WAIT_PEER : FP_WAIT_LOCAL)) {
            fail(cx, 0x20000 | (tag & 0x1ff));   // the hidden state of this phase never arrived
            break;
        }
    }
    double s = 0.0;
    float amax = 0.0f;   // max |x_j * gamma_j|: with the norm's factor it bounds the result
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const __half2* gh2 = reinterpret_cast<const __half2*>(&gm[e]);
#pragma unroll
        for (int k = 0; k < 2; ++k) {   // chunks past the end are zero
            const uint32_t pw = (uint32_t)w[e][k];
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pw));
            const float2 gf = __half22float2(gh2[k]);
            s += (double)(f.x * f.x);
            s += (double)(f.y * f.y);
            amax = fmaxf(amax, fmaxf(fabsf(f.x * gf.x), fabsf(f.y * gf.y)));
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        s += shfl_xor_double(s, m);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    if (lane == 0) {   // (the row's readers of two calls ago are many barriers away)
        drow[warp] = s;
        row[2 * F_NW + warp] = amax;
    }
    __syncthreads();
    double tot = drow[lane & (F_NW - 1)];
    amax = row[2 * F_NW + (lane & (F_NW - 1))];
#pragma unroll
    for (int m = 8; m > 0; m >>= 1) {
        tot += shfl_xor_double(tot, m);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    const float mean_sq = __fdiv_rn((float)tot, (float)H);                          // Inference.cu:136
    const float denom = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, p.eps)));     // Inference.cu:137
    const __half nscale = __float2half_rn(denom);                                   // Inference.cu:138
    // |fp16(fp16(x * nscale) * gamma)| <= |x * gamma| * nscale * (1 + 2^-11)^2 (+ half a subnormal step)
    bound = amax * __half2float(nscale) * 1.002f + 1e-7f;
    const XScale xq = xscale_for(bound);
    float ps[2] = {0.0f, 0.0f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int ch = tid + e * FP_NT;
        if (ch < nch) {
            const uint32_t p0 = (uint32_t)w[e][0], p1 = (uint32_t)w[e][1];
            const __half2 xa = *reinterpret_cast<const __half2*>(&p0), xb = *reinterpret_cast<const __half2*>(&p1);
            const __half* gh = reinterpret_cast<const __half*>(&gm[e]);
            __half o[4];
            o[0] = h_mul(h_mul(__low2half(xa), nscale), gh[0]);             // Inference.cu:142-143
            o[1] = h_mul(h_mul(__high2half(xa), nscale), gh[1]);
            o[2] = h_mul(h_mul(__low2half(xb), nscale), gh[2]);
            o[3] = h_mul(h_mul(__high2half(xb), nscale), gh[3]);
            if (QUANT) {
                uint32_t ph = 0u, pm = 0u, pl = 0u;
                int sum = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int X = xfix(o[k], xq);
                    xdigits(X, k, ph, pm, pl);
                    sum += X;
                }
                *reinterpret_cast<uint32_t*>(cx.xd + 4 * ch) = ph;
                *reinterpret_cast<uint32_t*>(cx.xd + FP_MAX_H + 4 * ch) = pm;
                *reinterpret_cast<uint32_t*>(cx.xd + 2 * FP_MAX_H + 4 * ch) = pl;
                ps[e] = (float)sum * xq.inv;
            } else {
                uint2 ov;
                ov.x = pack_h2(o[0], o[1]);
                ov.y = pack_h2(o[2], o[3]);
                *reinterpret_cast<uint2*>(out + 4 * ch) = ov;
                ps[e] = (__half2float(o[0]) + __half2float(o[1])) + (__half2float(o[2]) + __half2float(o[3]));
            }
        }
    }
    if (QUANT && tid == 0) *cx.xinv = xq.inv;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ps[e] += __shfl_xor_sync(0xffffffffu, ps[e], m);
        if (lane == 0) row[e * F_NW + warp] = ps[e];
    }
    __syncthreads();   // the result and the warp sums are visible
    x_full = 0.0f;
    x_slice = 0.0f;
    const int lo = slice * hs, hi = lo + hs;
#pragma unroll
    for (int k = 0; k < 2 * F_NW; ++k) {
        const float v = row[k];
        x_full += v;
        const int first = 4 * ((k & (F_NW - 1)) * 32 + (k / F_NW) * FP_NT);   // first element of that warp's row of chunks
        if (first >= lo && first < hi) x_slice += v;                           // (slice < 0: the range is empty)
    }
}

// This CTA's rs elements of the residual stream (hmine) as tagged words into buffer `buf` of every rank's copy.
template <bool SYS>
__device__ __forceinline__ void publish_hidden(const FusedParams& p, const FCtx& cx, const int buf, const uint32_t tag, const int cglob) {
    const int tid = threadIdx.x;
    const FusedGeom& G = p.g;
    if (tid < (G.rs >> 1)) {
        const uint32_t pair = pack_h2(cx.hmine[2 * tid], cx.hmine[2 * tid + 1]);
        const size_t at = (size_t)buf * (G.H >> 1) + (size_t)((G.rs * cglob) >> 1) + tid;
        for (int r = 0; r < G.n_ranks; ++r) stt<SYS>(p.hid[r] + at, tagged(pair, tag));
    }
}

// ---- exchange inside a head group through distributed shared memory (the group is one thread-block cluster) --------------
// A value goes into the same slot of every member's shared memory by an asynchronous store that also counts its bytes
// off the member's barrier (st.async ... mbarrier::complete_tx), so no fence and no separate arrival follow: the first
// form of this exchange (plain remote stores, then a release arrival per warp on every member's barrier) took a
// microsecond longer than the tagged words in global memory it replaced.  A member arms its OWN barrier once per
// layer with the bytes it expects, waits on it (one lane per warp polls, bounded) and reads its own shared memory.
__device__ __forceinline__ uint32_t cl_map(uint32_t addr, int cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cl_store(const float* slot, float v, uint32_t bar, int gs) {
    const uint32_t a = smem_u32(slot);
    for (int q = 0; q < gs; ++q)
        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                     ::"r"(cl_map(a, q)), "r"(__float_as_uint(v)), "r"(cl_map(bar, q)) : "memory");
}
__device__ __forceinline__ void cl_wait(const FCtx& cx, uint32_t bar, uint32_t parity, int code) {   // whole warps call
    if ((threadIdx.x & 31) == 0) {
        const long long t_begin = clock64();
        for (;;) {
            uint32_t ok;
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                         : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
            if (ok || *cx.s_dead != 0) break;
            if (clock64() - t_begin > FP_WAIT_LOCAL) {
                fail(cx, code);   // a member of the head group never delivered its part
                break;
            }
        }
    }
    __syncwarp();
}

// ---- one decoder layer for the CTAs that run the layers (runOneLayer, Inference.cu:1029-1230) -----------------------------
template <bool SYS>
__device__ __forceinline__ void layer_pass(const FusedParams& p, const FCtx& cx, WarpRing& ring, const int li) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, c = blockIdx.x;
    const FusedGeom& G = p.g;
    const FLayerDesc& L = cx.ldesc[li & 1];
    const float2* const lsz = cx.lsz + (li & 1) * 4 * FP_MAX_GROUPS;
    LayerPrefetch lp;
    layer_request(p, li + 1, lp);   // committed at the end of this layer
    const int H = G.H, gs = G.gs, rs = G.rs, n1 = G.n1;
    const int h_l = c / gs, r = c % gs, hglob = G.rank * G.heads_local + h_l, cglob = G.rank * G.n_act + c;
    const int hs = H / gs;
    const int pos = cx.pos;
    const uint32_t t0 = cx.tagbase + 2 + 6 * li;                 // + 0 xq, 1 xa, 2 xo, 3 hid[0], 4 x2, 5 hid[1]
    const uint32_t tag_in = li == 0 ? cx.tagbase + 1 : t0 - 1;   // hid[1] of the embedding / of the layer before
    const int o_first = rs * cglob;                              // this CTA's part of the residual stream

    // ---- RMSNorm + this CTA's K-slice of Wqkv for its head (Inference.cu:1036-1065) -----------------------------------
    float x_full, x_slice, x_bound;
    FP_STAMP(li, 0);
    gather_norm<SYS, true>(p, cx, p.hid[G.rank] + (H >> 1), tag_in, L.gamma, nullptr, r, hs, x_full, x_slice, x_bound, 0);
    FP_STAMP(li, 1);
    float sc = 0.0f, zp = 0.0f;
    if (tid < FP_QKV) {
        const int tile = tid >> 4, row = tid & 15;
        const long long o = (long long)(tile >> 3) * H + hglob * 128 + (tile & 7) * 16 + row;
        group_consts(lsz + F_QKV * FP_MAX_GROUPS, o, sc, zp);
    }
    run_gemv(ring, F_QKV, cx.xd + r * hs);
    __syncthreads();
    FP_STAMP(li, 2);
    if (tid < FP_QKV) {
        const float S = sum_k_shares(cx, p.plan[F_QKV], tid);
        const float part = sc * (S - zp * x_slice);
        if (p.cluster) {
            cl_store(cx.xq_in + r * FP_QKV + tid, part, cx.cl_bars, gs);
        } else {
            stt<false>(p.xq + (size_t)c * FP_QKV + tid, tagged_f(part, t0));
        }
    }
    // ---- attention: cache rows of earlier positions are requested before q is known -----------------------------------
    // Very short contexts: every CTA of the head group runs over ALL positions and the exchange of the attention states
    // is skipped.  (From about a hundred positions on the split is faster: 1.233 against 1.249 ms per token at 133-153
    // positions, 1.305 against 1.408 at 517-537.)
    const int len = pos + 1;
    const bool split = gs > 1 && len > p.attn_split_min;
    const int chunk = split ? (len + gs - 1) / gs : len;
    const int p0 = split ? r * chunk : 0, p1 = min(len, p0 + chunk);
    if (p.cluster && tid == 0) {   // bytes the other members (and this CTA) will store into this CTA's slots in this layer
        mbar_expect_tx(cx.cl_bars, (uint32_t)gs * FP_QKV * 4);
        if (split) mbar_expect_tx(cx.cl_bars + 8, (uint32_t)gs * 130 * 4);
    }
    const int grp = tid >> 4, sl = tid & 15;
    constexpr int NG = FP_NT / 16, UN = 2;
    const __half* kh = L.kc + (size_t)hglob * p.max_pos * 128 + sl * 8;
    const __half* vh = L.vc + (size_t)hglob * p.max_pos * 128 + sl * 8;
    uint4 nk[UN], nv[UN];
    auto request_rows = [&](const int kb) {
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int kp = kb + grp + u * NG;
            nk[u] = make_uint4(0u, 0u, 0u, 0u);
            nv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (kp < p1 && kp != pos) {
                nk[u] = __ldcg(reinterpret_cast<const uint4*>(kh + (size_t)kp * 128));
                nv[u] = __ldcg(reinterpret_cast<const uint4*>(vh + (size_t)kp * 128));
            }
        }
    };
    request_rows(p0);
    // ---- group exchange: q, k, v of the head = ordered sum of the gs K-slices; RoPE; KV append (Inference.cu:1070-1103)
    if (tid < FP_QKV) {
        float v = 0.0f;
        if (p.cluster) {
            cl_wait(cx, cx.cl_bars, li & 1, 0x30000 | li);
            for (int r0 = 0; r0 < gs; ++r0) v += cx.xq_in[r0 * FP_QKV + tid];
        } else {
            const unsigned long long* src = p.xq + (size_t)(h_l * gs) * FP_QKV + tid;
            for (int r0 = 0; r0 < gs; r0 += 4) {
                unsigned long long w[4];
                poll_batch<false, 4>(p, cx, gs - r0, [&](int e) { return src + (size_t)(r0 + e) * FP_QKV; }, t0, 0x30000 | li, w);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (r0 + e < gs) v += payload_f(w[e]);
            }
        }
        const int tile = tid >> 4, row = tid & 15, sec = tile >> 3, d = (tile & 7) * 16 + row;
        __half me = __float2half_rn(v);                                                       // Inference.cu:1062 (fp16 store)
        const __half other = __ushort_as_half((unsigned short)__shfl_xor_sync(0xffffffffu, (unsigned)__half_as_ushort(me), 1));
        if (sec < 2) {   // applyRotaryKernel, Inference.cu:150-177: pairs (2i, 2i+1)
            const __half cs = cx.rope_cs[d >> 1], sn = cx.rope_cs[64 + (d >> 1)];
            __half o0, o1;
            rope_pair((d & 1) ? other : me, (d & 1) ? me : other, cs, sn, o0, o1);
            me = (d & 1) ? o1 : o0;
        }
        cx.qkv_s[tid] = me;
        if (r == 0 && sec > 0) (sec == 1 ? L.kc : L.vc)[((size_t)hglob * p.max_pos + pos) * 128 + d] = me;   // Inference.cu:1094-1103
    }
    __syncthreads();
    FP_STAMP(li, 3);
    // ---- attention over positions [p0, p1) (attentionKernel, Inference.cu:182-266, intended math) -----------------------
    {
        float qf[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) qf[e] = __half2float(cx.qkv_s[sl * 8 + e]);
        const float scale = 1.0f / sqrtf(128.0f);
        float m = -INFINITY, l = 0.0f, ov[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) ov[e] = 0.0f;
        for (int kb = p0; kb < p1; kb += NG * UN) {   // trip count uniform across the CTA
            uint4 kv[UN], vv[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int kp = kb + grp + u * NG;
                kv[u] = nk[u];
                vv[u] = nv[u];
                if (kp < p1 && kp == pos) {   // this token's own row is not in the cache yet for the other CTAs of the group
                    kv[u] = *reinterpret_cast<const uint4*>(cx.qkv_s + 128 + sl * 8);
                    vv[u] = *reinterpret_cast<const uint4*>(cx.qkv_s + 256 + sl * 8);
                }
            }
            if (kb + NG * UN < p1) request_rows(kb + NG * UN);
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int kp = kb + grp + u * NG;
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
                if (kp < p1) {
                    const float s = dot * scale;
                    const float mn = fmaxf(m, s);
                    const float corr = (m == -INFINITY) ? 0.0f : expf(m - mn);
                    const float pr = expf(s - mn);
                    l = l * corr + pr;
                    const __half2* vh2 = reinterpret_cast<const __half2*>(&vv[u]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(vh2[e]);
                        ov[2 * e] = fmaf(pr, f.x, ov[2 * e] * corr);
                        ov[2 * e + 1] = fmaf(pr, f.y, ov[2 * e + 1] * corr);
                    }
                    m = mn;
                }
            }
        }
        // merge of the 32 half-warp states of the CTA in a fixed order
        float* st = cx.obuf;
#pragma unroll
        for (int e = 0; e < 8; ++e) st[grp * FP_ATT_STRIDE + sl * 8 + e] = ov[e];
        if (sl == 0) {
            st[grp * FP_ATT_STRIDE + 128] = m;
            st[grp * FP_ATT_STRIDE + 129] = l;
        }
        __syncthreads();
        float* wts = st + NG * FP_ATT_STRIDE;   // [NG] weights, then the maximum
        static_assert(NG == 32 && (NG + 1) * FP_ATT_STRIDE <= FP_OBUF, "one lane per half-warp state");
        if (tid < 32) {
            const float mg = st[tid * FP_ATT_STRIDE + 128];
            float mx = mg;
#pragma unroll
            for (int msk = 16; msk > 0; msk >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, msk));
            wts[tid] = (mg == -INFINITY) ? 0.0f : expf(mg - mx);
            if (tid == 0) wts[NG] = mx;
        }
        __syncthreads();
        float M = -INFINITY, Lsum = 0.0f, O = 0.0f;
        if (tid < 128) {
            M = wts[NG];
#pragma unroll 8
            for (int gq = 0; gq < NG; ++gq) {
                const float w = wts[gq];
                Lsum += st[gq * FP_ATT_STRIDE + 129] * w;
                O += st[gq * FP_ATT_STRIDE + tid] * w;
            }
        }
        FP_STAMP(li, 4);
        if (split) {
            // group exchange: every CTA of the head stores its state and merges all gs of them in CTA order
            const float* sts = st;   // the gs states to merge
            if (p.cluster) {         // they arrive in this CTA's own shared memory: the four warps that merge wait for them, no CTA barrier
                if (tid < 128) {
                    cl_store(cx.xa_in + r * FP_ATT_STRIDE + tid, O, cx.cl_bars + 8, gs);
                    if (tid == 0) {
                        cl_store(cx.xa_in + r * FP_ATT_STRIDE + 128, M, cx.cl_bars + 8, gs);
                        cl_store(cx.xa_in + r * FP_ATT_STRIDE + 129, Lsum, cx.cl_bars + 8, gs);
                    }
                    cl_wait(cx, cx.cl_bars + 8, li & 1, 0x40000 | li);
                }
                sts = cx.xa_in;
            } else {
                if (tid < 128) stt<false>(p.xa + (size_t)c * FP_ATT_STRIDE + tid, tagged_f(O, t0 + 1));
                if (tid == 0) {
                    stt<false>(p.xa + (size_t)c * FP_ATT_STRIDE + 128, tagged_f(M, t0 + 1));
                    stt<false>(p.xa + (size_t)c * FP_ATT_STRIDE + 129, tagged_f(Lsum, t0 + 1));
                }
                __syncthreads();   // everybody has read st
                if (tid < 130) {
                    const unsigned long long* src = p.xa + (size_t)(h_l * gs) * FP_ATT_STRIDE + tid;
                    for (int r0 = 0; r0 < gs; r0 += 4) {
                        unsigned long long w[4];
                        poll_batch<false, 4>(p, cx, gs - r0, [&](int e) { return src + (size_t)(r0 + e) * FP_ATT_STRIDE; }, t0 + 1,
                                             0x40000 | li, w);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (r0 + e < gs) st[(r0 + e) * FP_ATT_STRIDE + tid] = payload_f(w[e]);
                    }
                }
                __syncthreads();
            }
            if (tid < 128) {
                M = -INFINITY;
                for (int q = 0; q < gs; ++q) M = fmaxf(M, sts[q * FP_ATT_STRIDE + 128]);
                Lsum = 0.0f;
                O = 0.0f;
                for (int q = 0; q < gs; ++q) {
                    const float mq = sts[q * FP_ATT_STRIDE + 128];
                    const float w = (mq == -INFINITY) ? 0.0f : expf(mq - M);
                    Lsum += sts[q * FP_ATT_STRIDE + 129] * w;
                    O += sts[q * FP_ATT_STRIDE + tid] * w;
                }
            }
        }
        __half ch = __float2half_rn(0.0f);
        if (tid < 128) ch = __float2half_rn(O / Lsum);   // one rounding to fp16, Inference.cu:257-265
        float x_o, c_max;
        block_sum_max(cx, 0, __half2float(ch), fabsf(__half2float(ch)), x_o, c_max);   // its barrier also frees st
        quantise_own(cx, ch, 128, c_max);
        __syncthreads();
        FP_STAMP(li, 5);

        // ---- Wo restricted to the head's 128 inputs, this CTA's share of the outputs (Inference.cu:1122-1141) ----------
        const FGemvPlan& plo = p.plan[F_WO];
        run_gemv(ring, F_WO, cx.xd);
        __syncthreads();
        FP_STAMP(li, 6);
        const int n_out = plo.n_mt * 16;   // = hs
        for (int i0 = 2 * tid; i0 < n_out; i0 += 2 * FP_NT) {
            const long long o = (long long)r * hs + i0;
            float s2, z2;
            group_consts(lsz + F_WO * FP_MAX_GROUPS, o, s2, z2);
            const float y0 = s2 * (sum_k_shares(cx, plo, i0) - z2 * x_o), y1 = s2 * (sum_k_shares(cx, plo, i0 + 1) - z2 * x_o);
            const int ro = p.hpr_shift >= 0 ? (int)(o >> p.hpr_shift) : (int)(o / (H / G.n_ranks));   // rank that owns these two elements
            stt2<SYS>(p.xo[ro] + (size_t)(hglob * gs + r) * n_out + i0, tagged_f(y0, t0 + 2), tagged_f(y1, t0 + 2));
        }
        // ---- ordered sum over the heads for this CTA's rs outputs + residual (Inference.cu:1145-1156) ----------------------
        // The gathered words go to the end of obuf; where that does not overlap Wo's sums no barrier is needed in between.
        const int xo_at = (plo.wk * n_out + G.heads * rs <= FP_OBUF) ? FP_OBUF - G.heads * rs : 0;
        if (xo_at == 0) __syncthreads();   // obuf is free again
        float* const xo_s = cx.obuf + xo_at;
        {
            const int r_src = o_first / n_out, off = o_first % n_out;
            const int np = (G.heads * rs) >> 1;   // pairs of adjacent words: rs is even and a contributor's rs words are contiguous
            unsigned long long w[4][2];
            const unsigned long long* src = p.xo[G.rank] + (size_t)r_src * n_out + off;
            poll_pairs<SYS, 4>(p, cx, (np - tid + FP_NT - 1) / FP_NT,
                               [&](int e) {
                                   const int k = 2 * (tid + e * FP_NT), hq = p.rs_shift >= 0 ? k >> p.rs_shift : k / rs;
                                   return src + (size_t)hq * gs * n_out + (k - hq * rs);
                               }, t0 + 2,
                               0x50000 | li, w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (tid + e * FP_NT < np)
                    *reinterpret_cast<float2*>(xo_s + 2 * (tid + e * FP_NT)) = make_float2(payload_f(w[e][0]), payload_f(w[e][1]));
        }
        __syncthreads();
        FP_STAMP(li, 7);
        if (tid < rs) {
            float v = 0.0f;
            for (int hg = 0; hg < G.heads; ++hg) v += xo_s[hg * rs + tid];
            cx.hmine[tid] = h_add(cx.hmine[tid], __float2half_rn(v));   // fp16 store of the GEMV, then __hadd
        }
        if (rs <= 32) __syncwarp(); else __syncthreads();   // writers and readers of hmine are the first rs threads
        publish_hidden<SYS>(p, cx, 0, t0 + 3, cglob);
        FP_STAMP(li, 8);
    }

    if (c < G.n_mlp) {
    const int cmlp = G.rank * G.n_mlp + c;
    // ---- RMSNorm (same gamma) + this CTA's n1 outputs of W1 + GeLU (Inference.cu:1158-1197) ----------------------------------
    gather_norm<SYS, true>(p, cx, p.hid[G.rank], t0 + 3, L.gamma, nullptr, -1, H, x_full, x_slice, x_bound, 1);
    FP_STAMP(li, 9);
    if (tid < n1) group_consts(lsz + F_W1 * FP_MAX_GROUPS, (long long)cmlp * n1 + tid, sc, zp);
    run_gemv(ring, F_W1, cx.xd);
    __syncthreads();
    __half ge = __float2half_rn(0.0f);
    if (tid < n1) ge = gelu_h(__float2half_rn(sc * (sum_k_shares(cx, p.plan[F_W1], tid) - zp * x_full)));
    float x_g, g_max;
    block_sum_max(cx, 1, __half2float(ge), fabsf(__half2float(ge)), x_g, g_max);   // its barrier also frees obuf
    quantise_own(cx, ge, n1, g_max);
    __syncthreads();
    FP_STAMP(li, 10);
    // ---- W2 restricted to those n1 inputs, all outputs (Inference.cu:1198-1214) ------------------------------------------------
    run_gemv(ring, F_W2, cx.xd);
    __syncthreads();
    FP_STAMP(li, 11);
    for (int i0 = 2 * tid; i0 < H; i0 += 2 * FP_NT) {
        float s2, z2;
        group_consts(lsz + F_W2 * FP_MAX_GROUPS, i0, s2, z2);
        const float y0 = s2 * (cx.obuf[i0] - z2 * x_g), y1 = s2 * (cx.obuf[i0 + 1] - z2 * x_g);
        const int ro = p.hpr_shift >= 0 ? (i0 >> p.hpr_shift) : i0 / (H / G.n_ranks);
        stt2<SYS>(p.x2[ro] + (size_t)cmlp * H + i0, tagged_f(y0, t0 + 4), tagged_f(y1, t0 + 4));
    }
    __syncthreads();
    FP_STAMP(li, 14);
    }
    layer_commit(cx, (li + 1) & 1, lp);   // the next layer's constants: visible after the barriers below, last read a layer ago
    // ---- ordered sum over all contributors for this CTA's rs outputs + residual (Inference.cu:1217-1228) ----------------------
    const int ncontrib = G.n_ranks * G.n_mlp, nw = ncontrib * rs;
    if ((rs & 3) == 0) {   // a contributor's rs words are contiguous: four at a time
        const int nq4 = nw >> 2;
        unsigned long long w[2][4];
        const unsigned long long* src = p.x2[G.rank] + o_first;
        poll_quads<SYS, 2>(p, cx, (nq4 - tid + FP_NT - 1) / FP_NT,
                           [&](int e) {
                               const int k = 4 * (tid + e * FP_NT), cq = p.rs_shift >= 0 ? k >> p.rs_shift : k / rs;
                               return src + (size_t)cq * H + (k - cq * rs);
                           }, t0 + 4, 0x60000 | li, w);
#pragma unroll
        for (int e = 0; e < 2; ++e)
            if (tid + e * FP_NT < nq4)
                *reinterpret_cast<float4*>(cx.obuf + 4 * (tid + e * FP_NT)) =
                    make_float4(payload_f(w[e][0]), payload_f(w[e][1]), payload_f(w[e][2]), payload_f(w[e][3]));
    } else {
        const int np = nw >> 1;
        unsigned long long w[4][2];
        const unsigned long long* src = p.x2[G.rank] + o_first;
        poll_pairs<SYS, 4>(p, cx, (np - tid + FP_NT - 1) / FP_NT,
                           [&](int e) {
                               const int k = 2 * (tid + e * FP_NT), cq = p.rs_shift >= 0 ? k >> p.rs_shift : k / rs;
                               return src + (size_t)cq * H + (k - cq * rs);
                           }, t0 + 4, 0x60000 | li, w);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (tid + e * FP_NT < np)
                *reinterpret_cast<float2*>(cx.obuf + 2 * (tid + e * FP_NT)) = make_float2(payload_f(w[e][0]), payload_f(w[e][1]));
    }
    __syncthreads();
    FP_STAMP(li, 12);
    const int parts = (ncontrib % 4 == 0 && nw + 4 * rs <= FP_OBUF && 4 * rs <= FP_NT) ? 4 : 1;
    if (tid < parts * rs) {
        const int part = tid / rs, idx = tid % rs, per = ncontrib / parts;
        float v = 0.0f;
        for (int cc = part * per; cc < (part + 1) * per; ++cc) v += cx.obuf[cc * rs + idx];
        cx.obuf[nw + part * rs + idx] = v;
    }
    __syncthreads();
    if (tid < rs) {
        float v = cx.obuf[nw + tid];
        for (int q = 1; q < parts; ++q) v += cx.obuf[nw + q * rs + tid];
        cx.hmine[tid] = h_add(cx.hmine[tid], __float2half_rn(v));
    }
    if (rs <= 32) __syncwarp(); else __syncthreads();
    publish_hidden<SYS>(p, cx, 1, t0 + 5, cglob);
    FP_STAMP(li, 13);
    (void)lane; (void)warp;
}

// ---- final norm + unembedding + arg-max (sampleNextToken, Inference.cu:1235-1292) ---------------------------------------------
template <bool SYS>
__device__ __forceinline__ void sample_pass(const FusedParams& p, const FCtx& cx, WarpRing& ring) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, c = blockIdx.x;
    const FusedGeom& G = p.g;
    const int H = G.H, Kb = H >> 7, Mb = G.vocab >> 7;
    const uint32_t tag_in = p.n_layers > 0 ? cx.tagbase + 2 + 6 * (p.n_layers - 1) + 5 : cx.tagbase + 1;
    if (c >= G.n_act) {
        // CTAs without a part in the layers wait here for the whole pass: one thread polls, gently
        if (tid == 0) {
            const long long t_begin = clock64();
            while (!has_tag(ldt<SYS>(p.hid[G.rank] + (H >> 1)), tag_in) && *cx.s_dead == 0) {
                if (clock64() - t_begin > FP_WAIT_PEER) {
                    fail(cx, 0x70000);
                    break;
                }
                __nanosleep(1000);
            }
        }
        __syncthreads();
    }
    float xf, xsl, hv_bound;
    gather_norm<SYS, false>(p, cx, p.hid[G.rank] + (H >> 1), tag_in, p.gamma_final, cx.hv, -1, H, xf, xsl, hv_bound, 0);
    const int n_alloc = p.n_alloc[F_UNEMB];
    const int n_used = min(Kb, n_alloc);
    if (tid < n_used) cx.un_sz[tid] = pack_h2(p.un_scale[tid], p.un_zp[tid]);
    __syncthreads();
    // |x'_j| = |fp16(scale * x_j)| <= largest |scale| * bound of x (+ rounding): one fixed-point scale serves every round
    float smax = 0.0f;
    for (int k = 0; k < n_used; ++k) smax = fmaxf(smax, fabsf(__half2float(__ushort_as_half((unsigned short)(cx.un_sz[k] & 0xffffu)))));
    const XScale xq = xscale_for(hv_bound * smax * 1.001f + 1e-7f);
    if (tid == 0) *cx.xinv = xq.inv;
    const FGemvPlan& pl = p.plan[F_UNEMB];
    const int mstep = Mb % Kb;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int round = 0; round < p.n_rounds; ++round) {
        const long long blk = fused_unemb_block(G, c, round);
        if (blk < 0) break;
        // x'_j = scale[g(blk, j)] * x_j and Z = sum_j zp[g(blk, j)] * x'_j,  g(b, j) = ((b + j * Mb) mod Kb) mod entries
        // (the groups repeat with period Kb along j: entry r of this round's table serves every j = r mod Kb)
        const int bmod = (int)(blk % Kb);
        uint32_t* gtab = cx.un_sz + 64;
        if (tid < Kb) gtab[tid] = cx.un_sz[((bmod + tid * mstep) % Kb) % n_alloc];
        __syncthreads();
        const bool kb_pow2 = (Kb & (Kb - 1)) == 0;
        float zacc = 0.0f;
        for (int ch = tid; ch < (H >> 3); ch += FP_NT) {
            const uint4 xv = *reinterpret_cast<const uint4*>(cx.hv + 8 * ch);
            const __half* xh = reinterpret_cast<const __half*>(&xv);
            uint32_t ph[2] = {0u, 0u}, pm[2] = {0u, 0u}, pl[2] = {0u, 0u};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int j = 8 * ch + e;
                const uint32_t sz = gtab[kb_pow2 ? (j & (Kb - 1)) : (j % Kb)];
                const int X = xfix(h_mul(__ushort_as_half((unsigned short)(sz & 0xffffu)), xh[e]), xq);
                xdigits(X, e & 3, ph[e >> 2], pm[e >> 2], pl[e >> 2]);
                zacc = fmaf(__half2float(__ushort_as_half((unsigned short)(sz >> 16))), (float)X * xq.inv, zacc);
            }
            *reinterpret_cast<uint2*>(cx.xd + 8 * ch) = make_uint2(ph[0], ph[1]);
            *reinterpret_cast<uint2*>(cx.xd + FP_MAX_H + 8 * ch) = make_uint2(pm[0], pm[1]);
            *reinterpret_cast<uint2*>(cx.xd + 2 * FP_MAX_H + 8 * ch) = make_uint2(pl[0], pl[1]);
        }
        const float Z = block_sum_f(cx, zacc);   // its barriers also publish the digit planes
        run_gemv(ring, F_UNEMB, cx.xd);
        __syncthreads();
        if (tid < 128) {
            const __half hl = __float2half_rn(sum_k_shares(cx, pl, tid) - Z);   // fp16 logits, Inference.cu:1270
            const long long i = blk * 128 + tid;
            if (p.logits16) p.logits16[i] = hl;
            const float f = __half2float(hl);                                   // finalSoftmaxKernel, Inference.cu:284-292
            if (p.logits32) p.logits32[i] = f;
            if (f > best) {   // indices grow with the rounds: strict '>' keeps the first maximum (Inference.cu:1282-1289)
                best = f;
                besti = (int)i;
            }
        }
        __syncthreads();   // the digit planes and obuf are rewritten by the next round
    }
    // winner of this CTA, then of all CTAs of all ranks
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, m);
        if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) { cx.argv[warp] = best; cx.argi[warp] = besti; }
    __syncthreads();
    const uint32_t tag = cx.tagbase + 511;
    if (warp == 0) {
        best = lane < F_NW ? cx.argv[lane] : -INFINITY;
        besti = lane < F_NW ? cx.argi[lane] : 0x7fffffff;
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, m);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, m);
            if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
        }
        if (lane == 0) {
            const size_t at = 2 * (size_t)(G.rank * G.grid + c);
            for (int r = 0; r < G.n_ranks; ++r) stt2<SYS>(p.xarg[r] + at, tagged_f(best, tag), tagged((uint32_t)besti, tag));
        }
        if (c == 0) {
            const int n = G.n_ranks * G.grid;
            best = -INFINITY;
            besti = 0x7fffffff;
            for (int e = lane; e < n; e += 32) {
                unsigned long long a = 0, b = 0;
                const long long t_begin = clock64();
                for (;;) {
                    ldt2<SYS>(p.xarg[G.rank] + 2 * (size_t)e, a, b);
                    if ((has_tag(a, tag) && has_tag(b, tag)) || *cx.s_dead != 0) break;
                    if (clock64() - t_begin > (SYS ? FP_WAIT_PEER : FP_WAIT_LOCAL)) {
                        fail(cx, 0x80000);
                        break;
                    }
                }
                const float ov = payload_f(a);
                const int oi = (int)(uint32_t)b;
                if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, m);
                const int oi = __shfl_xor_sync(0xffffffffu, besti, m);
                if (better(ov, oi, best, besti)) { best = ov; besti = oi; }
            }
            if (lane == 0 && p.d_token_out) *p.d_token_out = besti;
        }
    }
}

// The shared-memory layout of the kernel (pointers only; the per-pass values tagbase / pos / n_seg are filled by the
// kernel, n_seg also lives in shared memory for the out-of-line GEMV).
__device__ __forceinline__ FCtx carve_ctx(uint8_t* smem) {
    FCtx cx;
    cx.ring = smem;
    cx.obuf = reinterpret_cast<float*>(smem + FP_OFF_OBUF);
    cx.hv = reinterpret_cast<__half*>(smem + FP_OFF_HV);
    cx.xd = smem + FP_OFF_XS;
    cx.xq_in = reinterpret_cast<float*>(smem + FP_OFF_CL);
    cx.xa_in = cx.xq_in + FP_CL_MAX * FP_QKV;
    cx.cl_bars = smem_u32(smem + FP_OFF_CL + (size_t)FP_CL_MAX * (FP_QKV + FP_ATT_STRIDE) * 4);
    cx.seg = reinterpret_cast<int4*>(smem + FP_OFF_SEG);
    cx.lsz = reinterpret_cast<float2*>(smem + FP_OFF_LSZ);
    uint8_t* misc = smem + FP_OFF_MISC;
    cx.qkv_s = reinterpret_cast<__half*>(misc);                  // 768
    cx.hmine = reinterpret_cast<__half*>(misc + 2048);           // 512
    cx.rope_cs = reinterpret_cast<__half*>(misc + 2560);         // 256
    cx.wsum = reinterpret_cast<float*>(misc + 2816);             // 256
    cx.dsum = reinterpret_cast<double*>(misc + 3072);            // 256: two rows of F_NW
    cx.un_sz = reinterpret_cast<uint32_t*>(misc + 5120);         // 512: groups in use | this round's table
    cx.argv = reinterpret_cast<float*>(misc + 3456);             // 64
    cx.argi = reinterpret_cast<int*>(misc + 3520);               // 64
    cx.s_dead = reinterpret_cast<int*>(misc + 3584);             // 16
    cx.xinv = reinterpret_cast<float*>(misc + 3600);             // 16
    cx.zero_addr = smem_u32(misc + 3616);                        // 32 zero bytes (16-byte aligned)
    cx.bars = smem_u32(misc + 3712);                             // FP_SLOTS * 8
    cx.ring_cnt = reinterpret_cast<int*>(misc + 3840);           // FP_SLOTS * 4
    cx.ring_issued = reinterpret_cast<int*>(misc + 3968);
    cx.ldesc = reinterpret_cast<FLayerDesc*>(misc + 4096);       // 2 descriptors
    static_assert(FP_SLOTS <= 16 && 4096 + 2 * sizeof(FLayerDesc) <= 5120 && 5120 + 512 <= FP_MISC_BYTES, "misc area");

    cx.err = *reinterpret_cast<int**>(misc + 5632);                // written by the kernel before the first use
    cx.n_seg = *reinterpret_cast<int*>(misc + 5640);
    cx.plans = reinterpret_cast<const FGemvPlan*>(misc + 5648);   // F_NOPS plans
    cx.wplan = reinterpret_cast<const int4*>(misc + 5888);        // F_NOPS * F_NW entries
    cx.bsm = reinterpret_cast<float*>(misc + 5888 + F_NOPS * F_NW * 16);
    cx.gsm = cx.bsm + 4 * F_NW;
    static_assert(5888 + F_NOPS * F_NW * 16 + (4 + 6) * F_NW * 4 <= FP_MISC_BYTES, "scratch rows in the misc area");
    static_assert(5648 + F_NOPS * sizeof(FGemvPlan) <= 5888 && 5888 + F_NOPS * F_NW * 16 <= FP_MISC_BYTES, "plans in the misc area");
    cx.tagbase = 0;
    cx.pos = 0;
    return cx;
}

template <bool SYS>
__global__ void __launch_bounds__(FP_NT, 1) fused_pass_kernel(const FusedParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    {   // what the out-of-line GEMV reads from shared memory: error word, segment count, operator plans
        uint8_t* misc0 = smem + FP_OFF_MISC;
        if (threadIdx.x == 0) {
            *reinterpret_cast<int**>(misc0 + 5632) = p.err;
            *reinterpret_cast<int*>(misc0 + 5640) = 4 * p.n_layers + p.n_rounds;
#ifdef QW3_TRACE
            *reinterpret_cast<unsigned long long**>(misc0 + 3680) = p.trace ? p.trace + (size_t)gridDim.x * p.n_layers * 16 : nullptr;
#endif
        }
        static_assert(sizeof(FGemvPlan) % 4 == 0 && 5648 + F_NOPS * sizeof(FGemvPlan) <= FP_MISC_BYTES, "plans in the misc area");
        for (int i = threadIdx.x; i < (int)(F_NOPS * sizeof(FGemvPlan) / 4); i += FP_NT)
            reinterpret_cast<int*>(misc0 + 5648)[i] = reinterpret_cast<const int*>(p.plan)[i];
        if (threadIdx.x < F_NOPS * F_NW) {   // what a warp derives from the plan, once instead of at every call
            const FGemvPlan& pl = p.plan[threadIdx.x / F_NW];
            const int warp = threadIdx.x % F_NW, a = warp / pl.wk, bk = warp % pl.wk;
            reinterpret_cast<int4*>(misc0 + 5888)[threadIdx.x] =
                make_int4(bk * (4 * pl.nq + pl.rem) * 16, bk * (pl.n_mt * 16) + a * (pl.nb * pl.tb) * 16, pl.rem ? 1 : pl.nq / pl.gu,
                          pl.rem ? pl.nq : pl.gu);
        }
        __syncthreads();
    }
    FCtx cx = carve_ctx(smem);
    uint32_t* zero = reinterpret_cast<uint32_t*>(smem + FP_OFF_MISC + 3616);
    const int tid = threadIdx.x, c = blockIdx.x;
    const FusedGeom& G = p.g;
    const bool active = c < G.n_act;
    const int cglob = G.rank * G.n_act + c;
    // this CTA's share of every weight stream, in the order of consumption
    for (int i = tid; i < cx.n_seg; i += FP_NT) {
        const uint8_t* base = nullptr;
        int wb = 0, ub = 1;
        if (i < 4 * p.n_layers) {
            const FGemvPlan& pl = p.plan[i & 3];
            ub = pl.unit_bytes;
            if (c < pl.n_cta) {
                wb = pl.warp_bytes;
                base = p.layers[i >> 2].d.w[i & 3] + (size_t)c * F_NW * wb;
            }
        } else {
            const int round = i - 4 * p.n_layers;
            ub = p.plan[F_UNEMB].unit_bytes;
            if (fused_unemb_block(G, c, round) >= 0) {
                wb = p.plan[F_UNEMB].warp_bytes;
                base = p.un_w + ((size_t)round * G.grid + c) * F_NW * wb;
            }
        }
        const unsigned long long b = reinterpret_cast<unsigned long long>(base);
        cx.seg[i] = make_int4((int)(uint32_t)b, (int)(uint32_t)(b >> 32), wb, ub);
    }
    if (tid == 0) {
        for (int s = 0; s < FP_SLOTS; ++s) {
            mbar_init(cx.bars + 8 * s, 1);
            cx.ring_cnt[s] = 0;
        }
        *cx.s_dead = 0;
        *cx.ring_issued = 0;
        if (p.cluster) {   // one arrival per layer: this CTA arming the barrier with the bytes it expects
            mbar_init(cx.cl_bars, 1);
            mbar_init(cx.cl_bars + 8, 1);
        }
        mbar_fence_init();
    }
    if (tid < 8) zero[tid] = 0u;
#ifdef QW3_TRACE
    if (tid == 0 && p.trace != nullptr && p.n_layers > 0) {   // which SM runs this CTA (slot 15 of its first layer's stamps)
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.trace[((size_t)blockIdx.x * p.n_layers) * 16 + 15] = smid;
    }
#endif
    cx.pos = __ldcg(p.d_pos);
    const int gen = p.d_gen != nullptr ? __ldcg(p.d_gen) : 0;
    cx.tagbase = (((uint32_t)gen & 0x3fu) << 26) | ((((uint32_t)cx.pos + 1u) & 0x1ffffu) << 9);
    if (tid < 64) {   // applyRotaryKernel's table row of this position (Inference.cu:444-454)
        cx.rope_cs[tid] = p.cos_t[(size_t)cx.pos * 64 + tid];
        cx.rope_cs[64 + tid] = p.sin_t[(size_t)cx.pos * 64 + tid];
    }
    __syncthreads();
    if (p.cluster) {   // every member's barriers exist before anybody arrives on them (the only unbounded wait: it is the first thing every CTA does)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (p.dry) return;
    WarpRing ring;
    ring.uc = 0; ring.pseg = 0; ring.pu = 0;
    for (int s = 0; s < FP_SLOTS; ++s) {   // prime the ring: thread 0 issues, every warp moves its cursor along
        if (ring_cursor_valid(ring, cx)) {
#ifndef QW3_FP_NOLOAD
            if (tid == 0) ring_issue(ring, cx, s);
#endif
            ++ring.pu;
        }
    }

    if (active) {
        {
            LayerPrefetch lp0;
            layer_request(p, 0, lp0);
            layer_commit(cx, 0, lp0);   // visible after the barrier below
        }
        // embedding gather (Inference.cu:1310-1315) or the hidden state the pass before left (Inference.cu:1357)
        if (tid < G.rs) {
            const int i = G.rs * cglob + tid;
            const bool keep = !p.first_stage || (p.d_skip != nullptr && __ldcg(p.d_skip) != 0);
            __half v;
            if (keep) {
                v = __ldcg(p.hidden + i);
            } else {
                long long tok = p.decode ? __ldcg(p.d_token) : __ldcg(p.d_prompt + cx.pos);
                if (tok < 0 || tok >= G.vocab) tok = 0;
                const long long pc = ((long long)G.vocab + 1) / 2;
                const long long gq = (tok / 128) % p.emb_n_alloc;
                const uint32_t byte = p.emb_packed[(long long)i * pc + (tok >> 1)];
                v = dequant_one((tok & 1) ? (byte >> 4) : (byte & 15u), p.emb_zp[gq], p.emb_scale[gq]);
            }
            cx.hmine[tid] = v;
        }
        __syncthreads();
        publish_hidden<SYS>(p, cx, 1, cx.tagbase + 1, cglob);
        for (int li = 0; li < p.n_layers; ++li) layer_pass<SYS>(p, cx, ring, li);
        if (tid < G.rs) p.hidden[G.rs * cglob + tid] = cx.hmine[tid];   // for the next pass / the next stage
        if (G.n_ranks > 1) {
            // Row-split over GPUs: the plain hidden state of this GPU is completed from the words the other GPUs'
            // CTAs of the same index published (readers after this launch expect the whole vector).
            const int half = G.rs >> 1, n = (G.n_ranks - 1) * half;
            const uint32_t tag = p.n_layers > 0 ? cx.tagbase + 2 + 6 * (p.n_layers - 1) + 5 : cx.tagbase + 1;
            if (tid < n) {
                int r = tid / half;
                r += r >= G.rank ? 1 : 0;
                const size_t at = (size_t)(((r * G.n_act + c) * G.rs) >> 1) + tid % half;
                unsigned long long w[1];
                poll_batch<SYS, 1>(p, cx, 1, [&](int) { return p.hid[G.rank] + (G.H >> 1) + at; }, tag, 0xA0000, w);
                reinterpret_cast<uint32_t*>(p.hidden)[at] = (uint32_t)w[0];
            }
        }
    }
    if (p.n_rounds > 0) sample_pass<SYS>(p, cx, ring);
    // After a wait has given up, units may have been requested that nobody consumed: their copies must have landed
    // before the CTA gives up its shared memory (bounded; a normal pass has none outstanding).
    __syncthreads();
    if (tid == 0 && *cx.s_dead != 0) {
        const int issued = *cx.ring_issued;
        for (int u = ring.uc; u < issued; ++u) {
            const long long t_begin = clock64();
            while (!mbar_try_wait(cx.bars + 8 * (u % FP_SLOTS), (u / FP_SLOTS) & 1) && clock64() - t_begin < (1ll << 24)) {}
        }
    }
}

// ---- load-time repack ------------------------------------------------------------------------------------------------------
// One 32-bit word of a stream: `stream` is the CTA (or, for the unembedding, round * grid + CTA), `warp` and `off` the
// position inside it.  raw: the matrix as on disk, element (o, j) = nibble (f & 1) of byte f >> 1, f = o + j * out_dim
// (the flat stream read column-major, Inference.cu:1052-1065 over Inference.cu:84-105).
QW3_HD uint32_t fused_repack_word(const FusedGeom& g, const FGemvPlan& pl, int op, const uint8_t* raw, long long out_dim,
                                  long long stream, int warp, int off) {
    const int cta = op == F_UNEMB ? (int)(stream % g.grid) : (int)stream;
    const long long blk = op == F_UNEMB ? fused_unemb_block(g, cta, (int)(stream / g.grid)) : 0;
    if (blk < 0) return 0u;
    const FWordPos wp = fused_word_pos(pl, warp, off);
    const long long o0 = fused_tile_out(g, op, cta, wp.tile, blk), k0 = fused_k0(g, op, cta);
    uint32_t word = 0u;
    for (int n = 0; n < 8; ++n) {
        int row, j;
        fused_nibble_src(wp, n, row, j);
        const long long f = (o0 + row) + (k0 + j) * out_dim;
        const uint32_t byte = raw[f >> 1];
        word |= ((f & 1) ? (byte >> 4) : (byte & 15u)) << (4 * n);
    }
    return word;
}

// Word `wi` of the repacked buffer: streams follow one another; inside a stream the units follow one another, a unit
// being [warp][piece] (fused_stream_locate, fused_plan.h).
__global__ void fused_repack_kernel(const FusedGeom g, const FGemvPlan pl, const int op, const uint8_t* __restrict__ raw,
                                    const long long out_dim, uint32_t* __restrict__ out, const long long n_words) {
    const long long wi = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= n_words) return;
    const long long wps = (long long)F_NW * pl.warp_bytes / 4;   // words per stream
    const long long stream = wi / wps;
    int warp, off;
    fused_stream_locate(pl, (int)(wi % wps) * 4, warp, off);
    out[wi] = fused_repack_word(g, pl, op, raw, out_dim, stream, warp, off);
}

// Fills the per-layer constant blocks from the descriptors (one block of FP_NT threads per layer): entry b of matrix k
// is the (scale, zero point) pair of its output block b, group = ((b mod (in_dim / 128)) mod entries).
__global__ void fused_consts_kernel(FLayerConst* lc, const int4 n_alloc, const int4 kb, const int4 mb) {
    FLayerConst& L = lc[blockIdx.x];
    const int tid = threadIdx.x, k = tid / FP_MAX_GROUPS, b = tid % FP_MAX_GROUPS;
    const int na = k == 0 ? n_alloc.x : k == 1 ? n_alloc.y : k == 2 ? n_alloc.z : n_alloc.w;
    const int kbk = k == 0 ? kb.x : k == 1 ? kb.y : k == 2 ? kb.z : kb.w;
    const int mbk = k == 0 ? mb.x : k == 1 ? mb.y : k == 2 ? mb.z : mb.w;
    uint32_t v = 0u;
    if (b < mbk) {
        const int gq = (b % kbk) % na;
        v = pack_h2(L.d.scale[k][gq], L.d.zp[k][gq]);
    }
    L.sz[k][b] = v;
}

// ---- host side ---------------------------------------------------------------------------------------------------------------
static bool make_plan(int n_cta, int n_mt, int n_ks, FGemvPlan* pl) {
    for (int wm = F_NW; wm >= 1; wm >>= 1) {
        if (n_mt % wm) continue;
        const int wk = F_NW / wm;
        if (n_ks % wk) continue;
        const int ksw = n_ks / wk, rem = ksw % 4, mtw = n_mt / wm;
        if (rem != 0 && rem != 2) continue;
        const int nq = ksw / 4;
        int tb = 0;
        for (int t = 4; t >= 1; --t)   // with a half group the whole block is one ring unit and must fit a slot
            if (mtw % t == 0 && (rem == 0 || (t % 2 == 0 && t * (nq * 512 + rem * 128) <= F_UNIT))) { tb = t; break; }
        if (tb == 0) continue;
        if ((long long)wk * n_mt * 16 > FP_OBUF) continue;
        pl->n_cta = n_cta; pl->n_mt = n_mt; pl->n_ks = n_ks; pl->wk = wk; pl->tb = tb; pl->nb = mtw / tb;
        pl->nq = nq; pl->rem = rem;
        pl->warp_bytes = pl->nb * tb * (nq * 512 + rem * 128);
        if (rem) {
            pl->gu = nq;
            pl->unit_bytes = tb * (nq * 512 + rem * 128);
        } else {
            int gu = 1;
            for (int c = 8; c >= 1; c >>= 1)
                if (nq % c == 0 && c * tb * 512 <= F_UNIT) { gu = c; break; }
            pl->gu = gu;
            pl->unit_bytes = gu * tb * 512;
        }
        pl->n_units = pl->warp_bytes / pl->unit_bytes;
        return true;
    }
    return false;
}

// group(b, j) = ((b + j * Mb) mod Kb) mod entries does not depend on j
static bool groups_uniform(long long M, long long K, long long n_alloc) {
    const long long Mb = M / 128, Kb = K / 128;
    for (long long b = 0; b < Mb; ++b)
        for (long long j = 1; j < Kb; ++j)
            if (((b + j * Mb) % Kb) % n_alloc != (b % Kb) % n_alloc) return false;
    return true;
}

bool fused_plan(int H, int I, int heads, int vocab, int n_layers, long long max_pos, int n_ranks, int rank, int grid,
                FusedGeom* geom, FGemvPlan* plans) {
    if (H <= 0 || heads <= 0 || H != heads * 128 || H > FP_MAX_H || H % 128 || I % 128 || vocab % 128) return false;
    if (n_ranks < 1 || n_ranks > QW3_MAX_STAGES || rank < 0 || rank >= n_ranks || heads % n_ranks) return false;
    if (grid < 1 || max_pos > 0x1fffe || 6 * n_layers + 8 >= 511) return false;
    if (3 * H / 128 > FP_MAX_GROUPS || I / 128 > FP_MAX_GROUPS) return false;
    FusedGeom g;
    g.H = H; g.I = I; g.heads = heads; g.vocab = vocab; g.n_ranks = n_ranks; g.rank = rank; g.grid = grid;
    g.heads_local = heads / n_ranks;
    g.n_blocks = vocab / 128;
    bool found = false;
    for (int gs = 32; gs >= 1 && !found; gs >>= 1) {
        const int n_act = g.heads_local * gs;
        if (n_act > grid || H % gs || (H / gs) % 128 || gs * FP_ATT_STRIDE > FP_OBUF) continue;
        if (H % (n_ranks * n_act)) continue;
        const int rs = H / (n_ranks * n_act);
        if (rs < 2 || rs % 2 || rs > FP_MAX_RS || (H / gs) % rs || (H / n_ranks) % rs) continue;
        // W1 / W2: as many of the n_act CTAs as give every one a multiple of 32 outputs of W1 (its k-steps of W2 then
        // come in pairs); with the matrices row-split over many GPUs fewer CTAs than n_act take part
        int n1 = 0, n_mlp = 0;
        for (int cand = 32; cand <= FP_MAX_N1 && cand <= FP_NT; cand += 32) {
            if (I % (n_ranks * cand)) continue;
            const int m = I / (n_ranks * cand);
            if (m <= n_act && m > n_mlp) { n_mlp = m; n1 = cand; }
        }
        if (n_mlp == 0) continue;
        if ((H / gs) % 2 || (long long)heads * rs > 8 * FP_NT || (long long)n_ranks * n_mlp * rs > 8 * FP_NT) continue;
        g.gs = gs; g.n_act = n_act; g.rs = rs; g.n1 = n1; g.n_mlp = n_mlp;
        FGemvPlan pl[F_NOPS];
        if (!make_plan(n_act, 24, H / 16 / gs, &pl[F_QKV])) continue;
        if (!make_plan(n_act, H / gs / 16, 8, &pl[F_WO])) continue;
        if (!make_plan(g.n_mlp, n1 / 16, H / 16, &pl[F_W1])) continue;
        if (!make_plan(g.n_mlp, H / 16, n1 / 16, &pl[F_W2])) continue;
        if (!make_plan(grid, 8, H / 16, &pl[F_UNEMB])) continue;
        for (int k = 0; k < F_NOPS; ++k) plans[k] = pl[k];
        found = true;
    }
    if (!found) return false;
    const int n_rounds = (g.n_blocks + n_ranks * grid - 1) / (n_ranks * grid);
    if (4 * n_layers + n_rounds > FP_MAX_SEG) return false;
    // the layer matrices must have groups that depend on the output only (they do for the reference's shapes)
    if (!groups_uniform(3LL * H, H, 3LL * H / 128) || !groups_uniform(H, H, H / 128) || !groups_uniform(I, H, I / 128) ||
        !groups_uniform(H, I, H / 128))
        return false;
    *geom = g;
    return true;
}

size_t fused_stream_bytes(const FusedGeom& g, const FGemvPlan& pl, int op) {
    const long long streams = op == F_UNEMB ? (long long)((g.n_blocks + g.n_ranks * g.grid - 1) / (g.n_ranks * g.grid)) * g.grid : pl.n_cta;
    return (size_t)streams * F_NW * pl.warp_bytes;
}

void fused_repack_host(const FusedGeom& g, const FGemvPlan& pl, int op, const uint8_t* raw, long long out_dim, uint8_t* out) {
    const size_t bytes = fused_stream_bytes(g, pl, op);
    const long long wps = (long long)F_NW * pl.warp_bytes / 4;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
    for (size_t wi = 0; wi < bytes / 4; ++wi) {
        const long long stream = (long long)(wi / wps);
        int warp, off;
        fused_stream_locate(pl, (int)(wi % wps) * 4, warp, off);
        o32[wi] = fused_repack_word(g, pl, op, raw, out_dim, stream, warp, off);
    }
}

struct FusedPass {
    FusedParams prm;
    std::vector<void*> allocs;
    int device = 0;
    int grid = 0;
    bool sys = false;
    void* xbase = nullptr;        // this rank's exchange buffers (one allocation, exported to the peers when row-split)
    size_t xoff[4] = {0, 0, 0, 0};
};

static int fp_alloc(FusedPass* f, void** p, size_t bytes) {
    cudaError_t r = cudaMalloc(p, bytes);
    if (r != cudaSuccess) {
        set_last_error("cudaMalloc(%zu bytes) for the fused pass -> %s", bytes, cudaGetErrorString(r));
        return r == cudaErrorMemoryAllocation ? QW3_ERR_NOMEM : QW3_ERR_CUDA;
    }
    f->allocs.push_back(*p);
    return QW3_OK;
}

#define FP_TRY(expr)                      \
    do {                                  \
        int rc__ = (expr);                \
        if (rc__ != QW3_OK) return rc__;  \
    } while (0)

static int repack_to_device(FusedPass* f, const FusedGeom& g, const FGemvPlan& pl, int op, const FusedMatrix& m, const uint8_t** out,
                            cudaStream_t st) {
    const size_t bytes = fused_stream_bytes(g, pl, op);
    void* d = nullptr;
    FP_TRY(fp_alloc(f, &d, bytes));
    const long long n_words = (long long)(bytes / 4);
    const long long blocks = (n_words + 255) / 256;
    fused_repack_kernel<<<(unsigned)blocks, 256, 0, st>>>(g, pl, op, static_cast<const uint8_t*>(m.packed), m.out_dim,
                                                          static_cast<uint32_t*>(d), n_words);
    QW3_CUDA(cudaGetLastError());
    *out = static_cast<const uint8_t*>(d);
    return QW3_OK;
}

// Sizes of the four exchange buffers that other ranks store into (xo, x2, hid, xarg), in 64-bit words.
static void exchange_words(const FusedGeom& g, size_t (&w)[4]) {
    w[0] = (size_t)g.heads * g.gs * (g.H / g.gs);
    w[1] = (size_t)g.n_ranks * g.n_mlp * g.H;
    w[2] = (size_t)g.H;   // two buffers of H / 2
    w[3] = 2 * (size_t)g.n_ranks * g.grid;
}

// Cooperative launch of `grid` CTAs; cluster > 0: in thread-block clusters of that many CTAs.
static void fused_launch_config(int grid, int cluster, cudaStream_t st, cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(grid);
    cfg->blockDim = dim3(FP_NT);
    cfg->dynamicSmemBytes = FP_SMEM_BYTES;
    cfg->stream = st;
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
    if (cluster > 0) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cluster;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg->numAttrs = 2;
    }
}

int fused_create(const FusedCreate& a, FusedPass** out) {
    FusedPass* f = new (std::nothrow) FusedPass();
    if (!f) return QW3_ERR_NOMEM;
    f->device = a.device;
    f->grid = a.sm_count;
    FusedParams& P = f->prm;
    std::memset(&P, 0, sizeof(P));
    auto bail = [&](int rc) {
        fused_destroy(f);
        return rc;
    };
    if (!fused_plan(a.H, a.I, a.heads, a.vocab, a.n_layers, a.max_pos, a.n_ranks, a.rank, a.sm_count, &P.g, P.plan)) {
        set_last_error("the fused pass does not support this configuration");
        return bail(QW3_ERR_ARG);
    }
    const FusedGeom& g = P.g;
    cudaError_t ce = cudaFuncSetAttribute(fused_pass_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FP_SMEM_BYTES);
    if (ce == cudaSuccess) ce = cudaFuncSetAttribute(fused_pass_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FP_SMEM_BYTES);
    int nb = 0;
    if (ce == cudaSuccess) ce = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fused_pass_kernel<false>, FP_NT, FP_SMEM_BYTES);
    if (ce != cudaSuccess || nb < 1) {
        set_last_error("fused_pass_kernel does not fit on an SM (%zu bytes of shared memory): %s", FP_SMEM_BYTES, cudaGetErrorString(ce));
        return bail(QW3_ERR_CUDA);
    }
    // One GPU, head groups of 2 .. FP_CL_MAX CTAs: the group becomes a thread-block cluster and exchanges through
    // distributed shared memory, when the device can hold enough clusters at once for the CTAs that run the layers.
    // (The grid is then a multiple of the cluster size, so the plan is made again for that grid.)
    if (g.n_ranks == 1 && g.gs >= 2 && g.gs <= FP_CL_MAX && !a.no_cluster) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        fused_launch_config(a.sm_count - a.sm_count % g.gs, g.gs, a.stream, &cfg, attr);
        int n_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, fused_pass_kernel<false>, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n_clusters = 0;
        }
        const int grid_c = std::min(a.sm_count - a.sm_count % g.gs, n_clusters * g.gs);
        if (grid_c >= g.n_act) {
            const int gs_before = g.gs;
            FusedGeom g2;
            FGemvPlan pl2[F_NOPS];
            if (fused_plan(a.H, a.I, a.heads, a.vocab, a.n_layers, a.max_pos, a.n_ranks, a.rank, grid_c, &g2, pl2) && g2.gs == gs_before) {
                P.g = g2;
                for (int k = 0; k < F_NOPS; ++k) P.plan[k] = pl2[k];
                f->grid = grid_c;
                P.cluster = 1;
            }
        }
    }
    P.n_layers = a.n_layers;
    P.eps = a.eps;
    P.attn_split_min = a.attn_split_min;
    auto log2_exact = [](int v) {
        int sh = 0;
        while ((1 << sh) < v) ++sh;
        return (1 << sh) == v ? sh : -1;
    };
    P.hpr_shift = log2_exact(g.H / g.n_ranks);
    P.rs_shift = log2_exact(g.rs);
    P.n_rounds = a.unemb ? (g.n_blocks + g.n_ranks * g.grid - 1) / (g.n_ranks * g.grid) : 0;
    P.first_stage = a.emb ? 1 : 0;
    std::vector<FLayerConst> ld((size_t)a.n_layers);
    for (int l = 0; l < a.n_layers; ++l) {
        const FusedLayerIn& in = a.layers[l];
        std::memset(&ld[l], 0, sizeof(FLayerConst));
        for (int k = 0; k < 4; ++k) {
            int rc = repack_to_device(f, g, P.plan[k], k, in.m[k], &ld[l].d.w[k], a.stream);
            if (rc != QW3_OK) return bail(rc);
            ld[l].d.scale[k] = static_cast<const __half*>(in.m[k].scale);
            ld[l].d.zp[k] = static_cast<const __half*>(in.m[k].zp);
            if (l == 0) P.n_alloc[k] = (int)in.m[k].n_alloc;
            if (in.m[k].n_alloc > FP_MAX_GROUPS || in.m[k].n_alloc != P.n_alloc[k]) {
                set_last_error("the fused pass keeps at most %d scale / zero-point entries per layer matrix", FP_MAX_GROUPS);
                return bail(QW3_ERR_ARG);
            }
        }
        ld[l].d.gamma = static_cast<const __half*>(in.gamma);
        ld[l].d.kc = static_cast<__half*>(in.kc);
        ld[l].d.vc = static_cast<__half*>(in.vc);
    }
    void* d_layers = nullptr;
    int rc = fp_alloc(f, &d_layers, sizeof(FLayerConst) * (size_t)(a.n_layers > 0 ? a.n_layers : 1));
    if (rc != QW3_OK) return bail(rc);
    if (a.n_layers > 0) {
        // pageable source: the copy is staged before the call returns
        if (cudaMemcpyAsync(d_layers, ld.data(), sizeof(FLayerConst) * ld.size(), cudaMemcpyHostToDevice, a.stream) != cudaSuccess)
            return bail(QW3_ERR_CUDA);
        fused_consts_kernel<<<a.n_layers, FP_NT, 0, a.stream>>>(
            static_cast<FLayerConst*>(d_layers), make_int4(P.n_alloc[0], P.n_alloc[1], P.n_alloc[2], P.n_alloc[3]),
            make_int4(a.H / 128, a.H / 128, a.H / 128, a.I / 128), make_int4(3 * a.H / 128, a.H / 128, a.I / 128, a.H / 128));
        if (cudaGetLastError() != cudaSuccess) return bail(QW3_ERR_CUDA);
    }
    P.layers = static_cast<const FLayerConst*>(d_layers);
    if (a.emb) {
        P.emb_packed = static_cast<const uint8_t*>(a.emb->packed);
        P.emb_scale = static_cast<const __half*>(a.emb->scale);
        P.emb_zp = static_cast<const __half*>(a.emb->zp);
        P.emb_n_alloc = (int)a.emb->n_alloc;
    }
    if (a.unemb) {
        rc = repack_to_device(f, g, P.plan[F_UNEMB], F_UNEMB, *a.unemb, &P.un_w, a.stream);
        if (rc != QW3_OK) return bail(rc);
        P.un_scale = static_cast<const __half*>(a.unemb->scale);
        P.un_zp = static_cast<const __half*>(a.unemb->zp);
        P.n_alloc[F_UNEMB] = (int)a.unemb->n_alloc;
        P.gamma_final = static_cast<const __half*>(a.gamma_final);
        P.logits16 = static_cast<__half*>(a.logits16);
        P.logits32 = a.logits32;
    }
    P.hidden = static_cast<__half*>(a.hidden);
    P.d_pos = a.d_pos; P.d_token = a.d_token; P.d_skip = a.d_skip; P.d_prompt = a.d_prompt; P.d_gen = a.d_gen;
    P.cos_t = static_cast<const __half*>(a.cos_t); P.sin_t = static_cast<const __half*>(a.sin_t);
    P.max_pos = a.max_pos;
    P.d_token_out = a.d_token;
    P.err = a.err;
    // exchange buffers: the group-local ones, then one allocation for those other ranks store into
    void* loc = nullptr;
    const size_t loc_words = (size_t)g.n_act * (FP_QKV + FP_ATT_STRIDE);
    rc = fp_alloc(f, &loc, loc_words * 8);
    if (rc != QW3_OK) return bail(rc);
    if (cudaMemsetAsync(loc, 0, loc_words * 8, a.stream) != cudaSuccess) return bail(QW3_ERR_CUDA);
    P.xq = static_cast<unsigned long long*>(loc);
    P.xa = P.xq + (size_t)g.n_act * FP_QKV;
    size_t w[4];
    exchange_words(g, w);
    size_t total = 0;
    for (int k = 0; k < 4; ++k) {
        f->xoff[k] = total;
        total += (w[k] + 31) & ~(size_t)31;
    }
    rc = fp_alloc(f, &f->xbase, total * 8);
    if (rc != QW3_OK) return bail(rc);
    if (cudaMemsetAsync(f->xbase, 0, total * 8, a.stream) != cudaSuccess) return bail(QW3_ERR_CUDA);
    if (cudaStreamSynchronize(a.stream) != cudaSuccess) return bail(QW3_ERR_CUDA);
    fused_set_peer(f, g.rank, f->xbase);
#ifdef QW3_TRACE
    {
        void* tr = nullptr;
        const size_t tb = ((size_t)f->grid * (a.n_layers > 0 ? a.n_layers : 1) * 16 + 2048) * 8;   // + 1024 unit waits of CTA 0
        rc = fp_alloc(f, &tr, tb);
        if (rc != QW3_OK) return bail(rc);
        cudaMemset(tr, 0, tb);
        P.trace = static_cast<unsigned long long*>(tr);
    }
#endif
    f->sys = g.n_ranks > 1;
    if (P.cluster) {
        // Occupancy said the clusters fit; a launch that does nothing proves it (a profiler, or another client of the GPU,
        // can leave too few SMs for co-resident clusters).  If it is refused the same grid runs without clusters: the head
        // groups then exchange through global memory, as they do when the matrices are row-split over GPUs.
        FusedParams q = P;
        q.dry = 1;
        void* args[] = {&q};
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        fused_launch_config(f->grid, g.gs, a.stream, &cfg, attr);
        cudaError_t le = cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(fused_pass_kernel<false>), args);
        if (le == cudaSuccess) le = cudaStreamSynchronize(a.stream);
        if (le != cudaSuccess) {
            (void)cudaGetLastError();
            P.cluster = 0;
        }
    }
    *out = f;
    return QW3_OK;
}

void* fused_exchange_base(FusedPass* f, size_t* bytes) {
    size_t w[4];
    exchange_words(f->prm.g, w);
    if (bytes) *bytes = (f->xoff[3] + ((w[3] + 31) & ~(size_t)31)) * 8;
    return f->xbase;
}

// Exchange buffers of rank r (its own allocation, or a peer mapping of another rank's).
void fused_set_peer(FusedPass* f, int r, void* base) {
    unsigned long long* b = static_cast<unsigned long long*>(base);
    f->prm.xo[r] = b + f->xoff[0];
    f->prm.x2[r] = b + f->xoff[1];
    f->prm.hid[r] = b + f->xoff[2];
    f->prm.xarg[r] = b + f->xoff[3];
}

void fused_destroy(FusedPass* f) {
    if (!f) return;
    for (void* p : f->allocs) cudaFree(p);
    delete f;
}

int fused_launch(FusedPass* f, int decode, cudaStream_t st) {
    FusedParams p = f->prm;
    p.decode = decode;
    if (!decode) p.n_rounds = 0;   // prompt passes compute no logits (Inference.cu:1304-1343)
    void* args[] = {&p};
    const void* fn = f->sys ? reinterpret_cast<const void*>(fused_pass_kernel<true>) : reinterpret_cast<const void*>(fused_pass_kernel<false>);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    fused_launch_config(f->grid, p.cluster ? p.g.gs : 0, st, &cfg, attr);
    QW3_CUDA(cudaLaunchKernelExC(&cfg, fn, args));
    return QW3_OK;
}

// Tracing builds: the stamps of the last pass, [grid][n_layers][16] (null otherwise).
const void* fused_trace(const FusedPass* f, size_t* bytes) {
    if (bytes) *bytes = ((size_t)f->grid * (f->prm.n_layers > 0 ? f->prm.n_layers : 1) * 16 + 2048) * 8;
    return f->prm.trace;
}

void fused_geometry(const FusedPass* f, FusedGeom* g, FGemvPlan* plans) {
    *g = f->prm.g;
    for (int k = 0; k < F_NOPS; ++k) plans[k] = f->prm.plan[k];
}

}  // namespace qw3

using namespace qw3;

extern "C" {

int qw3_fused_plan(const Qw3Config* cfg, int32_t n_ranks, int32_t rank, int32_t grid, int32_t* geom_out, int32_t* plans_out) {
    QW3_REQUIRE(cfg && geom_out && plans_out, "qw3_fused_plan: null pointer");
    FusedGeom g;
    FGemvPlan pl[F_NOPS];
    if (!fused_plan(cfg->hidden, cfg->inter, cfg->heads, cfg->vocab, cfg->layers, cfg->max_pos, n_ranks, rank, grid, &g, pl)) {
        set_last_error("qw3_fused_plan: the fused pass does not cover this configuration");
        return QW3_ERR_ARG;
    }
    const int32_t gv[16] = {g.H, g.I, g.heads, g.vocab, g.n_ranks, g.rank, g.heads_local, g.gs, g.n_act, g.rs, g.n1, g.n_blocks, g.grid, g.n_mlp, 0, 0};
    std::memcpy(geom_out, gv, sizeof(gv));
    for (int k = 0; k < F_NOPS; ++k) {
        const int32_t pv[10] = {pl[k].n_cta, pl[k].n_mt, pl[k].n_ks, pl[k].wk, pl[k].tb, pl[k].nb, pl[k].nq, pl[k].rem, pl[k].warp_bytes, pl[k].unit_bytes};
        std::memcpy(plans_out + 10 * k, pv, sizeof(pv));
    }
    return QW3_OK;
}

int qw3_fused_repack_host(const Qw3Config* cfg, int32_t n_ranks, int32_t rank, int32_t grid, int32_t op, const void* raw_packed,
                          int64_t out_dim, void* out, int64_t out_bytes) {
    QW3_REQUIRE(cfg && raw_packed && out && op >= 0 && op < F_NOPS, "qw3_fused_repack_host: bad argument");
    FusedGeom g;
    FGemvPlan pl[F_NOPS];
    if (!fused_plan(cfg->hidden, cfg->inter, cfg->heads, cfg->vocab, cfg->layers, cfg->max_pos, n_ranks, rank, grid, &g, pl)) {
        set_last_error("qw3_fused_repack_host: the fused pass does not cover this configuration");
        return QW3_ERR_ARG;
    }
    QW3_REQUIRE((int64_t)fused_stream_bytes(g, pl[op], op) == out_bytes, "qw3_fused_repack_host: the stream of this operator has %zu bytes",
                fused_stream_bytes(g, pl[op], op));
    fused_repack_host(g, pl[op], op, static_cast<const uint8_t*>(raw_packed), out_dim, static_cast<uint8_t*>(out));
    return QW3_OK;
}

}  // extern "C"
