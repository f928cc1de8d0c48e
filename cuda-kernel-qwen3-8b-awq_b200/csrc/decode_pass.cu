// One persistent kernel per token pass of a pipeline stage (sm_100a).
//
// The reference runs a token through a stage as 12 launches + 68 memcpys per layer with the host
// in the loop (runOneLayer, Inference.cu:1029-1230; generateResponse, Inference.cu:1304-1405).  At
// batch 1 every operator of the path moves a few tens of MB, which HBM delivers in 1-4 us: launch
// boundaries, not bytes, set the pace.  Here a whole pass -- embedding gather, then per layer
// RMSNorm+Wqkv+RoPE+KV append, attention, Wo+residual, RMSNorm+W1+GeLU, W2+residual, and on the
// last stage final norm + unembed + arg-max -- is one cooperative launch of one CTA per SM that
// walks a list of operator descriptors:
//   * the packed weights of ALL operators, in order, flow through one ring of 4 KB TMA boxes
//     (32 units, 128 KB per SM).  There is no producer warp: each of the 16 warps owns two ring
//     slots and, as soon as it has consumed a unit, issues the TMA load of the unit that will
//     land in the same slot 32 units later -- possibly a unit of a later operator, since weights
//     never depend on activations.  The ring is therefore full again by the time the warps have
//     crossed an operator boundary, and no empty-slot barrier exists;
//   * the warps take units round-robin (no stage-wide lock-step), unpack and accumulate exactly
//     as the stand-alone GEMV does, and reduce across warps once per tile in a fixed order;
//   * everything that crosses CTAs inside the launch travels as tagged 64-bit words -- (payload, tag) in
//     one aligned store, tag = launch epoch * 1024 + operator index -- which the reader polls: seeing the
//     tag means having the value, so there is no flag, fence or second round trip, and nothing is cleared
//     between launches.  Partial sums of a tile shared by several CTAs: every contributor stores its sums
//     and later gathers, for its own share of the tile's outputs, the words of all contributors in CTA
//     order (deterministic) and runs the epilogue there.  Activations: the epilogue stores (two halves,
//     tag) per output pair, the next operator's prologue polls them.  The only arrival counter left
//     precedes the final arg-max.  All CTAs are co-resident (cooperative launch), so the polls cannot
//     deadlock; every poll gives up after about a second and reports a located error word;
//   * with one process per GPU the same words cross NVLink (copyHiddenBetweenGPUs, Inference.cu:1013-1023, without
//     a launch or a host wait): the last residual operator of a stage stores its tagged output with system scope
//     into the next GPU's inbox, the first operators of the next stage poll that inbox in their own memory, and the
//     arg-max stores (id, tag) into the first stage's token word, which its embedding polls.  Those words carry a
//     tag made of the generation counter and the token position, which all stages share; the waits are bounded
//     (about nine seconds) and the kernels that wait on one another run on different GPUs.
// Plain activations written inside the kernel (for readers after the launch) are never read back in it.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "pass_flags.h"

namespace qw3 {

constexpr int P_TI = WS_TILE;            // outputs per tile
constexpr int P_ROW_BYTES = P_TI / 2;    // 512
constexpr int P_UNIT_ROWS = 8;
constexpr int P_UNIT_BYTES = P_UNIT_ROWS * P_ROW_BYTES;   // 4096
constexpr int P_NCW = 16;                // 4 warps per scheduler: 128 registers per thread
constexpr int P_NCONS = P_NCW * 32;
constexpr int P_NTHREADS = P_NCONS;
constexpr int P_RING = 32;               // units in flight per SM (128 KB): two slots per warp
constexpr int P_MAXK = 12288;            // largest in_dim (activation vector kept in shared memory)
constexpr int P_MAXK_NU = 4096;          // largest in_dim of an operator with j-dependent groups
constexpr int P_MAX_GROUPS = 256;
constexpr int P_RED_BYTES = 65536;       // cross-warp reduction (16 slots x 4 KB) / 32 attention states (16.9 KB)
constexpr int P_OPW = 48;                // 32-bit words of a descriptor after its tensor map
constexpr int P_DONE = 256;              // largest number of tiles / heads of an operator
constexpr int P_MAX_OPS = 256;           // operators of one pass (their unit ranges are cached in shared memory)
constexpr int P_PSLOTS = WS_MAX_CTAS + P_DONE;   // partial-sum slots (CTA + tile) of an operator

constexpr size_t P_OFF_RED = (size_t)P_RING * P_UNIT_BYTES;
constexpr size_t P_OFF_XS = P_OFF_RED + P_RED_BYTES;
constexpr size_t P_OFF_GIDX = P_OFF_XS + (size_t)P_MAXK_NU * 2;   // inside xs: operators that use it have K <= P_MAXK_NU
constexpr size_t P_OFF_GTAB = P_OFF_XS + (size_t)P_MAXK * 2;
static_assert(2 * P_MAXK_NU <= P_MAXK, "the per-row group indices must fit behind the input vector");
constexpr size_t P_OFF_MISC = P_OFF_GTAB + (size_t)P_MAX_GROUPS * 16;
constexpr size_t P_OFF_RNG = P_OFF_MISC + 2048;                 // per-operator unit range of this CTA
constexpr size_t P_SMEM_BYTES = P_OFF_RNG + (size_t)P_MAX_OPS * 16;

enum PassOpKind { PASS_EMBED = 0, PASS_GEMV = 1, PASS_ATTN = 2 };

struct PassOpBody {          // 192 bytes, copied to shared memory per operator
    int32_t kind, uniform, exact, epilogue;
    int32_t M, K, Mb, Kb;
    int32_t n_alloc, n_tiles, upt, flags;
    long long U;
    const __half* scale;
    const __half* zp;
    const __half* x;         // plain input (used when xt is null)
    const __half* gamma;
    __half* y;
    __half* kc;
    __half* vc;
    const uint8_t* packed;   // embedding only
    float eps;
    int32_t src;             // operator that writes xt in this launch (its tag is expected in every word)
    // Activations between operators of one launch travel as tagged words: (two halves, tag) in one 64-bit
    // word per output pair, polled by the consumer, so no flag, fence or arrival counter sits between them.
    const unsigned long long* xt;   // tagged input, K/2 words (null: plain x)
    unsigned long long* yt;         // tagged copy of the output (null: none)
    const unsigned long long* rt;   // RESIDUAL: tagged words holding the value to add to (null: plain y)
    int32_t rsrc;                   // operator that wrote rt in this launch
    int32_t reserved1;
    long long reserved[4];
};
static_assert(sizeof(PassOpBody) == 192, "descriptor body must be 192 bytes");

struct alignas(128) PassOp {
    CUtensorMap tmap;
    PassOpBody b;
};
static_assert(sizeof(PassOp) == 384, "descriptor must be 384 bytes");

struct PassParams {
    const PassOp* ops;
    int n_ops;
    int* done;                // [n_ops] arrival counters (one arrival per CTA and operator), zeroed before the launch
    unsigned long long* xchg; // [2][P_PSLOTS][1024] tagged partial sums: operator parity, (CTA, tile) slot c + tile
    const int* d_epoch;       // launches completed on this stage so far (incremented after each pass); this launch
                              // writes *d_epoch + 1 into its flags, so flags never need clearing
    const int* d_pos;
    const int* d_token;       // sampled id of the previous step (decode pass)
    const int* d_skip;        // non-zero: keep the hidden state, skip the gather
    const int* d_prompt;      // prompt ids (prompt pass)
    int decode;
    const __half* cos_t;
    const __half* sin_t;
    int heads, hidden;
    long long max_pos, vocab;
    int* d_token_out;
    // One process per GPU, stages chained inside the kernels (no hand-off launches between passes): words that cross
    // GPUs carry a tag made of the generation counter and the token position, which every stage knows.
    const int* d_gen;                         // generation counter of this sequence (null: 0)
    const unsigned long long* tok_in;         // first stage: (sampled id, peer tag) stored by the last stage
    unsigned long long* const* tok_out_slot;  // last stage: device word holding the first stage's tok_in address (or null)
    float* logits_f32;
    unsigned long long* trace2;  // optional [grid][n_ops][8]: per-CTA event times inside each operator (debug)
    unsigned long long* trace;   // optional [n_ops + 1]: global timer when CTA 0 enters each operator
    Workspace ws;
};

// Tracing builds (-DQW3_TRACE) record global-timer stamps inside every operator; other builds hold none of this code.
__device__ __forceinline__ void trace_event(const PassParams& p, int o, int ev) {
#ifdef QW3_TRACE
    if (p.trace2 != nullptr && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace2[((size_t)blockIdx.x * p.n_ops + o) * 8 + ev] = t;
    }
#else
    (void)p; (void)o; (void)ev;
#endif
}

__device__ __forceinline__ void red_add_release(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Partial sums cross CTAs as (value, tag) words: the tag names the launch and the operator, value and tag
// travel in ONE aligned 64-bit store, so a reader that sees the tag has the value.
__device__ __forceinline__ unsigned long long pack_tagged(float v, uint32_t tag) {
    return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
}
__device__ __forceinline__ void st_relaxed_v2(unsigned long long* p, unsigned long long a, unsigned long long b) {
    asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_relaxed_v2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long a) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long a;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}
// The same single-word hand-over between GPUs (the writer is a kernel on the stage before / after): system scope.
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long a) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long a;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}
__device__ __forceinline__ void ld_relaxed_sys_v2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// Tag of a word that crosses GPUs: bit 31 (no launch tag has it while the epoch is below 2^21), the generation
// counter and the position + 1.  The words of an inbox are rewritten for every token, so the newest content always
// belongs to this position or to an earlier one of this or the previous generation.
__device__ __forceinline__ uint32_t peer_tag(int gen, int pos) {
    return 0x80000000u | (((uint32_t)gen & 0x3ffu) << 21) | (((uint32_t)pos + 1u) & 0x1fffffu);
}
// Waits on another GPU are bounded more generously than waits inside a launch (the stages run one after another).
constexpr long long P_PEER_WAIT_CLOCKS = 1ll << 34;
// Output pairs of a tile shared by CTAs cf..cl are dealt evenly: CTA c finalises pairs [pb, pe) of the
// 512; thread t of it takes pair pb + t.  Returns whether thread t has a pair.
__device__ __forceinline__ bool slice_pair(int cf, int cl, int c, int t, int& pp) {
    const int n = cl - cf + 1, k = c - cf;
    const int pb = (P_TI / 2) * k / n, pe = (P_TI / 2) * (k + 1) / n;
    pp = pb + t;
    return t < pe - pb;
}

// Share of one operator's units for CTA c: a contiguous range [ub, ub + n) of absolute units
// (tile * upt + row unit).  With fewer tiles than CTAs every CTA works inside ONE tile (tile t is cut
// evenly among CTAs [t*G/nt, (t+1)*G/nt)), so it reduces across warps and CTAs once per operator;
// otherwise the flattened unit space is cut into G equal ranges.  cf..cl are the CTAs that
// contribute to tile `tile_q`.
__device__ __forceinline__ void cta_range(long long U, int upt, int n_tiles, int c, int& ub, int& n) {
    const int Gf = gridDim.x;
    if (n_tiles < Gf) {   // 32-bit arithmetic: tiles <= 256, CTAs <= 256, units per tile <= 1536
        const int t = ((c + 1) * n_tiles - 1) / Gf;
        const int cb = t * Gf / n_tiles, cb1 = (t + 1) * Gf / n_tiles;
        const int cnt = min(cb1 - cb, upt), idx = c - cb;
        if (idx < cnt) {
            const int lo = idx * upt / cnt, hi = (idx + 1) * upt / cnt;
            ub = t * upt + lo;
            n = hi - lo;
        } else {
            ub = 0;
            n = 0;
        }
    } else {
        const int G = (long long)Gf < U ? Gf : (int)U;
        if (c < G) {
            const long long u0 = (long long)c * U / G, u1 = (long long)(c + 1) * U / G;
            ub = (int)u0;
            n = (int)(u1 - u0);
        } else {
            ub = 0;
            n = 0;
        }
    }
}
__device__ __forceinline__ void tile_contributors(long long U, int upt, int n_tiles, int tile, int& cf, int& cl) {
    const int Gf = gridDim.x;
    if (n_tiles < Gf) {
        const int cb = tile * Gf / n_tiles, cb1 = (tile + 1) * Gf / n_tiles;
        cf = cb;
        cl = cb + min(cb1 - cb, upt) - 1;
    } else {
        const int G = (long long)Gf < U ? Gf : (int)U;
        const long long ut0 = (long long)tile * upt;
        cf = owner_of(ut0, G, U);
        cl = owner_of(ut0 + upt - 1, G, U);
    }
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct PassSmem {
    const int4* s_rng;   // [n_ops] {first unit, units, units per tile, kind} of this CTA, filled at kernel start
    int* s_epoch;   // value this launch writes into its flags
    uint32_t* s_ptag;   // peer_tag(generation, position) of this pass
    uint8_t* ring;
    float* red;
    __half* xs;
    uint16_t* gidx;
    uint4* gtab;
    uint32_t full0;           // shared address of the ring barriers
    double* dsum;
    float* s_argv;
    int* s_argi;
    int* s_dead;
    uint32_t* s_op;           // [2][P_OPW]
};

// The operator before `o` must be complete before its outputs are read: every CTA arrives once per
// operator on its counter; thread 0 acquire-polls it (bounded), the CTA barrier hands the result on.
__device__ __forceinline__ void wait_for_previous(const PassParams& p, const PassSmem& sm, int o) {
    if (o > 0 && threadIdx.x == 0 && *sm.s_dead == 0) {
        const long long t0 = clock64();
        while (ld_acquire(p.done + o - 1) < (int)gridDim.x) {
            if (clock64() - t0 > (1ll << 31)) {
                atomicCAS(p.ws.err, 0, 0x20000 | o);   // operator o-1 never completed
                *sm.s_dead = 1;
                break;
            }
        }
    }
    named_barrier(1, P_NCONS);
    trace_event(p, o, 1);
}
// This CTA's part of operator o is written: one cumulative release after the CTA barrier.
__device__ __forceinline__ void publish(const PassParams& p, int o) {
    named_barrier(1, P_NCONS);
    if (threadIdx.x == 0) red_add_release(&p.done[o], 1);
}

// The chunks fetch_x3 is about to take, awaited with system-scope loads: their writer is the last operator of the
// stage before, on another GPU.  Not inlined: it runs once per pass, in the first operator of a stage.
__device__ __noinline__ void peer_wait_x3(const PassParams& p, const PassSmem& sm, const PassOpBody& op, const int o,
                                          const uint32_t xtag, const int first, const int limit) {
    const long long t_begin = clock64();
    for (;;) {
        bool ok = true;
        for (int e = 0; e < 3; ++e) {
            const int ch = first + e * P_NCONS;
            if (ch < limit) {
                unsigned long long a, b, c, d;
                ld_relaxed_sys_v2(op.xt + 4 * (size_t)ch, a, b);
                ld_relaxed_sys_v2(op.xt + 4 * (size_t)ch + 2, c, d);
                ok = ok && (uint32_t)(a >> 32) == xtag && (uint32_t)(b >> 32) == xtag && (uint32_t)(c >> 32) == xtag &&
                     (uint32_t)(d >> 32) == xtag;
            }
        }
        if (ok || *sm.s_dead != 0) return;
        if (clock64() - t_begin > P_PEER_WAIT_CLOCKS) {
            atomicCAS(p.ws.err, 0, 0x90000 | o);   // the stage before never delivered
            *sm.s_dead = 1;
            return;
        }
    }
}

// Up to three 16-byte chunks (8 halves each) of an operator's input vector for this thread: chunk indices
// first, first + 512, first + 1024 below `limit`.  Plain input: ordinary L2 loads.  Tagged input: every
// chunk is four (two halves, tag) words; all loads are in flight together and are repeated until every word
// carries the producer's tag (bounded).  (A one-word sentinel poll before the full fetch was measured: it
// costs one more L2 round trip per operator than it saves in polling traffic.)
__device__ __forceinline__ void fetch_x3(const PassParams& p, const PassSmem& sm, const PassOpBody& op, const int o,
                                         const uint32_t xtag, const int first, const int limit, uint4 (&xv)[3]) {
#pragma unroll
    for (int e = 0; e < 3; ++e) xv[e] = make_uint4(0u, 0u, 0u, 0u);
    if (op.xt == nullptr) {
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const int ch = first + e * P_NCONS;
            if (ch < limit) xv[e] = __ldcg(reinterpret_cast<const uint4*>(op.x) + ch);
        }
        return;
    }
    // Words the stage before stores from another GPU are first awaited with system-scope loads (bounded more
    // generously); the loop below then finds them at its first pass.  Kept out of the loop: the common case pays
    // one predicate.
    if (op.src == P_SRC_PEER) peer_wait_x3(p, sm, op, o, xtag, first, limit);
    const long long t_begin = clock64();
    __syncwarp();
    unsigned long long w[3][4] = {{0ull, 0ull, 0ull, 0ull}, {0ull, 0ull, 0ull, 0ull}, {0ull, 0ull, 0ull, 0ull}};
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const int ch = first + e * P_NCONS;
            if (ch < limit) {
                ld_relaxed_v2(op.xt + 4 * (size_t)ch, w[e][0], w[e][1]);
                ld_relaxed_v2(op.xt + 4 * (size_t)ch + 2, w[e][2], w[e][3]);
            }
        }
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            if (first + e * P_NCONS < limit) {
#pragma unroll
                for (int q = 0; q < 4; ++q) ok = ok && (uint32_t)(w[e][q] >> 32) == xtag;
            }
        }
        if (ok || *sm.s_dead != 0) break;
        if (clock64() - t_begin > (1ll << 31)) {
            atomicCAS(p.ws.err, 0, 0x20000 | o);
            *sm.s_dead = 1;
            break;
        }
    }
#pragma unroll
    for (int e = 0; e < 3; ++e)
        if (first + e * P_NCONS < limit) xv[e] = make_uint4((uint32_t)w[e][0], (uint32_t)w[e][1], (uint32_t)w[e][2], (uint32_t)w[e][3]);
}

// Per-warp prefetch cursor over the units this warp will consume (global unit counter uc = warp
// mod 16), walking through the operator list ahead of the computation.
struct Prefetch {
    int op;      // operator the cursor is in (-1 before the first)
    int uc;      // global unit counter of the last unit issued
    int base;    // global unit counter of the first unit of `op` for this CTA
    int n;       // units of `op` for this CTA
    int ub;      // first unit of this CTA in `op` (tile * upt + row unit)
    int upt;
    int next_u, tile, r;   // last unit issued in `op` and its (tile, row unit)
    bool end;
    uint64_t policy;       // L2 eviction policy of the weight stream
};

__device__ __forceinline__ void prefetch_next(Prefetch& pf, const PassParams& p, const PassSmem& sm) {
    if (pf.end) return;
    pf.uc += P_NCW;
    while (pf.uc - pf.base >= pf.n) {
        pf.base += pf.n;
        pf.n = 0;
        do {
            ++pf.op;
        } while (pf.op < p.n_ops && sm.s_rng[pf.op].w != PASS_GEMV);
        if (pf.op >= p.n_ops) {
            pf.end = true;
            return;
        }
        const int4 rg = sm.s_rng[pf.op];
        pf.ub = rg.x;
        pf.n = rg.y;
        pf.upt = rg.z;
        pf.next_u = pf.ub;
        pf.tile = pf.ub / pf.upt;
        pf.r = pf.ub - pf.tile * pf.upt;
    }
    // (tile, r) of unit ub + (uc - base), advanced incrementally from the last unit issued in this operator
    const int u = pf.ub + (pf.uc - pf.base);
    pf.r += u - pf.next_u;
    pf.next_u = u;
    while (pf.r >= pf.upt) {
        pf.r -= pf.upt;
        ++pf.tile;
    }
    const int tile = pf.tile, r = pf.r;
    if ((threadIdx.x & 31) == 0) {
        const int slot = pf.uc & (P_RING - 1);
        const uint32_t bar = sm.full0 + 8 * slot;
        // the slot was read by this warp with ordinary loads: order them before the bulk write
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, P_UNIT_BYTES);
        tma_load_2d_hint(smem_u32(sm.ring + slot * P_UNIT_BYTES), &p.ops[pf.op].tmap, tile * (P_TI / 8), r * P_UNIT_ROWS, bar,
                         pf.policy);
    }
}

// ---------------------------------------------------------------------------------------------
// Fused dequantise + matrix-vector product of one operator, for this CTA's share of its units.
// ---------------------------------------------------------------------------------------------
template <bool UNIFORM, bool EXACT>
__device__ __forceinline__ void gemv_phase(const PassParams& p, const PassOpBody& op, const int o, const PassSmem& sm,
                                            int& uc_base, const int pos, Prefetch& pf) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x;
    const long long U = op.U;
    const int upt = op.upt, K = op.K;
    const int u_begin = sm.s_rng[o].x, n_units = sm.s_rng[o].y;
    const int t0 = u_begin / upt, r0 = u_begin - t0 * upt;
    __half* xs = sm.xs;

    // ---- loads that do not depend on the previous operator are issued before waiting for it:
    // group constants of the first tile
    const int n_chunks = K >> 3;   // 16-byte chunks of 8 halves
    DqConst ku_first = {0u, 0u, 0u};
    if (UNIFORM) {
        int ib = t0 * (P_TI / 128) + (lane >> 2);
        if (ib >= op.Mb) ib = 0;
        const int g = (ib % op.Kb) % op.n_alloc;
        ku_first = make_const<EXACT>(op.zp[g], op.scale[g]);
    }
    if (op.flags & PASS_WAIT_PREV) wait_for_previous(p, sm, o);
    else trace_event(p, o, 1);
    const uint32_t xtag = op.src == P_SRC_PEER ? *sm.s_ptag : (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)op.src;
    const uint32_t tag = (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)o;
    // what the epilogue of the first tile will need (written two or more operators ago)
    uint32_t pre_a = 0u, pre_b = 0u;   // RESIDUAL: y[i], y[i+1];  ROPE_KV: cos, sin of this thread's pair
    if (n_units > 0) {
        int cf, cl, pp = tid;
        tile_contributors(U, upt, op.n_tiles, t0, cf, cl);
        const bool active = cf == cl ? true : slice_pair(cf, cl, c, tid, pp);
        const int i = t0 * P_TI + 2 * pp;
        if (active && i < op.M) {
            if (op.epilogue == QW3_EPI_RESIDUAL) {
                if (op.rt != nullptr) {   // value and tag; the tag is checked when the value is used
                    const unsigned long long w = ld_relaxed_u64(op.rt + (i >> 1));
                    pre_a = (uint32_t)w;
                    pre_b = (uint32_t)(w >> 32);
                } else {
                    pre_a = __ldcg(reinterpret_cast<const uint32_t*>(op.y + i));
                }
            } else if (op.epilogue == QW3_EPI_ROPE_KV && i < 2 * p.hidden) {
                const int d = i & 127;
                pre_a = __half_as_ushort(p.cos_t[(size_t)pos * 64 + (d >> 1)]);
                pre_b = __half_as_ushort(p.sin_t[(size_t)pos * 64 + (d >> 1)]);
            }
        }
    }

    // ---- epilogue of one output pair (outputs tile_e * 1024 + 2 * pp, + 1), called by all threads of the CTA
    auto epilogue = [&](const int tile_e, const int pp, const float v0, const float v1, const bool active) {
        const int i = tile_e * P_TI + 2 * pp;
        const bool valid = active && i < op.M;
        const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
        // plain store for readers after this launch; tagged copy for the next operator of this launch
        auto store_pair = [&](const __half a, const __half b) {
            const __half2 v = __halves2half2(a, b);
            *reinterpret_cast<__half2*>(op.y + i) = v;
            if (op.yt != nullptr) {
                // read here, not before the unit loop: nothing of the cross-GPU case stays live across the loop
                const bool peer_out = (op.flags & PASS_PEER_OUT) != 0;   // the tagged output goes to the next stage's GPU
                const uint32_t ytag = peer_out ? *sm.s_ptag : tag;
                const unsigned long long w = ((unsigned long long)ytag << 32) | *reinterpret_cast<const uint32_t*>(&v);
                if (peer_out) st_relaxed_sys_u64(op.yt + (i >> 1), w);
                else st_relaxed_u64(op.yt + (i >> 1), w);
            }
        };
        if (op.epilogue == QW3_EPI_STORE) {
            if (valid) store_pair(h0, h1);
        } else if (op.epilogue == QW3_EPI_RESIDUAL) {
            if (valid) {
                uint32_t rv;
                if (op.rt != nullptr) {
                    // the word must carry the tag of the operator that wrote the residual stream last: a CTA that
                    // had no part in the operators in between may be here before that word is written
                    // (residual stream of the stage before: its words were awaited with system-scope loads by this
                    // stage's first operator; the retry below repeats that if this CTA is ahead of it)
                    const bool rpeer = op.rsrc == P_SRC_PEER;
                    const uint32_t rtag = rpeer ? *sm.s_ptag : (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)op.rsrc;
                    unsigned long long w = tile_e == t0 ? (((unsigned long long)pre_b << 32) | pre_a) : ld_relaxed_u64(op.rt + (i >> 1));
                    const long long t_begin = clock64();
                    while ((uint32_t)(w >> 32) != rtag && *sm.s_dead == 0) {
                        if (clock64() - t_begin > (rpeer ? P_PEER_WAIT_CLOCKS : (1ll << 31))) {
                            atomicCAS(p.ws.err, 0, 0x80000 | o);   // the residual stream was never written
                            *sm.s_dead = 1;
                            break;
                        }
                        w = rpeer ? ld_relaxed_sys_u64(op.rt + (i >> 1)) : ld_relaxed_u64(op.rt + (i >> 1));
                    }
                    rv = (uint32_t)w;
                } else {
                    rv = tile_e == t0 ? pre_a : __ldcg(reinterpret_cast<const uint32_t*>(op.y + i));
                }
                const __half r0h = __ushort_as_half((unsigned short)(rv & 0xffffu)), r1h = __ushort_as_half((unsigned short)(rv >> 16));
                store_pair(h_add(r0h, h0), h_add(r1h, h1));
            }
        } else if (op.epilogue == QW3_EPI_GELU) {
            if (valid) store_pair(gelu_h(h0), gelu_h(h1));
        } else if (op.epilogue == QW3_EPI_ROPE_KV) {
            if (valid) {
                const int sec = i / p.hidden, idx = i - sec * p.hidden;
                const int head = idx >> 7, d = idx & 127;
                __half o0 = h0, o1 = h1;
                if (sec < 2) {
                    const __half cs = tile_e == t0 ? __ushort_as_half((unsigned short)pre_a) : p.cos_t[(size_t)pos * 64 + (d >> 1)];
                    const __half sn = tile_e == t0 ? __ushort_as_half((unsigned short)pre_b) : p.sin_t[(size_t)pos * 64 + (d >> 1)];
                    rope_pair(h0, h1, cs, sn, o0, o1);
                }
                __half* dst = sec == 0 ? op.y + idx : (sec == 1 ? op.kc : op.vc) + ((size_t)head * p.max_pos + pos) * 128 + d;
                const __half2 v = __halves2half2(o0, o1);
                *reinterpret_cast<__half2*>(dst) = v;
                if (op.yt != nullptr)   // q, k, v of this token as tagged words for the attention of this launch
                    st_relaxed_u64(op.yt + (i >> 1), ((unsigned long long)tag << 32) | *reinterpret_cast<const uint32_t*>(&v));
            }
        } else {  // QW3_EPI_ARGMAX: winner of this CTA's outputs of the tile -> slot c + tile_e
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            if (valid) {
                if (op.y) *reinterpret_cast<__half2*>(op.y + i) = __halves2half2(h0, h1);
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
            named_barrier(1, P_NCONS);   // the previous use of s_argv / s_argi is over
            if (lane == 0) { sm.s_argv[warp] = bv; sm.s_argi[warp] = bi; }
            named_barrier(1, P_NCONS);
            if (warp == 0) {
                bv = lane < P_NCW ? sm.s_argv[lane] : -INFINITY;
                bi = lane < P_NCW ? sm.s_argi[lane] : 0x7fffffff;
#pragma unroll
                for (int m = 8; m > 0; m >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                }
                if (lane == 0) {
                    p.ws.arg_val[c + tile_e] = bv;
                    p.ws.arg_idx[c + tile_e] = bi;
                }
            }
        }
    };
    int n_shared = 0, sh_tile0 = 0, sh_tile1 = 0;
    // Exchange slots alternate between two halves by operator parity: a slot is rewritten two operators later,
    // when every reader of this operator's words has provably finished.
    unsigned long long* const xchg_o = p.xchg + (size_t)(o & 1) * P_PSLOTS * P_TI;

    // ---- prologue: (RMS-normalised) input vector -> shared memory -------------------------------
    if (n_units == 0) {
        // nothing to multiply: the input is not read (a CTA that reads an input must also contribute to the
        // operator, so that nobody can run ahead and overwrite what it still reads)
    } else if (op.gamma != nullptr) {
        uint4 xv[3], gvv[3];
        double s = 0.0;
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const int ch = tid + e * P_NCONS;
            gvv[e] = make_uint4(0u, 0u, 0u, 0u);
            if (ch < n_chunks) gvv[e] = *(reinterpret_cast<const uint4*>(op.gamma) + ch);
        }
        fetch_x3(p, sm, op, o, xtag, tid, n_chunks, xv);
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const __half2* h = reinterpret_cast<const __half2*>(&xv[e]);
#pragma unroll
            for (int t = 0; t < 4; ++t) {   // chunks past the end are zero
                const float2 f = __half22float2(h[t]);
                s += (double)(f.x * f.x);
                s += (double)(f.y * f.y);
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) s += shfl_xor_double(s, m);
        if (lane == 0) sm.dsum[warp] = s;
        named_barrier(1, P_NCONS);
        double tot = sm.dsum[lane & (P_NCW - 1)];   // 16 partial sums: butterfly over the low four lane bits
#pragma unroll
        for (int m = 8; m > 0; m >>= 1) tot += shfl_xor_double(tot, m);
        const float mean_sq = __fdiv_rn((float)tot, (float)K);                         // Inference.cu:136
        const float denom = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, op.eps)));    // Inference.cu:137
        const __half nscale = __float2half_rn(denom);                                  // Inference.cu:138
#pragma unroll
        for (int e = 0; e < 3; ++e) {
            const int ch = tid + e * P_NCONS;
            if (ch < n_chunks) {
                const uint4 gv = gvv[e];
                const __half* xh = reinterpret_cast<const __half*>(&xv[e]);
                const __half* gh = reinterpret_cast<const __half*>(&gv);
                uint4 ov;
                __half* oh = reinterpret_cast<__half*>(&ov);
#pragma unroll
                for (int t = 0; t < 8; ++t) oh[t] = h_mul(h_mul(xh[t], nscale), gh[t]);  // Inference.cu:142-143
                *(reinterpret_cast<uint4*>(xs) + ch) = ov;
            }
        }
    } else if (n_units >= upt) {
        for (int base = 0; base < n_chunks; base += 3 * P_NCONS) {
            uint4 xv[3];
            fetch_x3(p, sm, op, o, xtag, base + tid, n_chunks, xv);
#pragma unroll
            for (int e = 0; e < 3; ++e)
                if (base + tid + e * P_NCONS < n_chunks) *(reinterpret_cast<uint4*>(xs) + base + tid + e * P_NCONS) = xv[e];
        }
    } else {
        // only the rows this CTA multiplies: [r0, r0 + n_units) units, wrapping once into the next tile
        const int a0 = r0, a1 = min(r0 + n_units, upt), b1 = r0 + n_units - upt;   // unit (= 16-byte chunk) ranges
        for (int base = a0; base < a1; base += 3 * P_NCONS) {
            uint4 xv[3];
            fetch_x3(p, sm, op, o, xtag, base + tid, a1, xv);
#pragma unroll
            for (int e = 0; e < 3; ++e)
                if (base + tid + e * P_NCONS < a1) *(reinterpret_cast<uint4*>(xs) + base + tid + e * P_NCONS) = xv[e];
        }
        for (int base = 0; base < b1; base += 3 * P_NCONS) {
            uint4 xv[3];
            fetch_x3(p, sm, op, o, xtag, base + tid, b1, xv);
#pragma unroll
            for (int e = 0; e < 3; ++e)
                if (base + tid + e * P_NCONS < b1) *(reinterpret_cast<uint4*>(xs) + base + tid + e * P_NCONS) = xv[e];
        }
    }
    if (!UNIFORM) {
        for (int j = tid; j < K; j += P_NCONS) sm.gidx[j] = (uint16_t)(((long long)j * op.Mb) % op.Kb);
        const int n_used = op.Kb < op.n_alloc ? op.Kb : op.n_alloc;
        for (int g = tid; g < n_used; g += P_NCONS) {
            const DqConst k = make_const<EXACT>(op.zp[g], op.scale[g]);
            sm.gtab[g] = make_uint4(k.z, k.hz, k.s, 0u);
        }
    }
    named_barrier(1, P_NCONS);
    trace_event(p, o, 2);

    float acc[4][2][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int d = 0; d < 4; ++d) acc[a][b][d] = 0.0f;

    const int q4 = lane >> 2, t4 = lane & 3;
    const bool is_b = (t4 == (q4 >> 1));
    const int bshift = (q4 & 1) * 16;

    int k = 0, tile = t0, r = r0;
    while (k < n_units) {
        const int seg = min(upt - r, n_units - k);
        DqConst ku = {0u, 0u, 0u};
        int ib = tile * (P_TI / 128) + (lane >> 2);
        if (ib >= op.Mb) ib = 0;               // columns past out_dim: zero-filled by TMA, results discarded
        const int ibk = ib % op.Kb;
        if (UNIFORM) {
            if (tile == t0) {
                ku = ku_first;
            } else {
                const int g = ibk % op.n_alloc;
                ku = make_const<EXACT>(op.zp[g], op.scale[g]);
            }
        }
        // ---- my units of this segment: those whose global counter is this warp's (mod 16)
        for (int kk = k + ((warp - uc_base - k) & (P_NCW - 1)); kk < k + seg; kk += P_NCW) {
            const int uc = uc_base + kk;
            const int slot = uc & (P_RING - 1);
            const uint32_t ph = (uc / P_RING) & 1;
            if (*sm.s_dead == 0 && !mbar_wait(sm.full0 + 8 * slot, ph)) {
                if (lane == 0) {
                    atomicCAS(p.ws.err, 0, 0x10000 | o);   // weights of operator o never arrived
                    *sm.s_dead = 1;
                }
            }
            const int row0 = (r + (kk - k)) * P_UNIT_ROWS;
            const uint8_t* ubase = sm.ring + slot * P_UNIT_BYTES + lane * 16;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int jrow = row0 + half * 4;
                const uint8_t* src = ubase + half * 4 * P_ROW_BYTES;
                const uint4 ra = *reinterpret_cast<const uint4*>(src);
                const uint4 rb = *reinterpret_cast<const uint4*>(src + P_ROW_BYTES);
                const uint4 rc = *reinterpret_cast<const uint4*>(src + 2 * P_ROW_BYTES);
                const uint4 rd = *reinterpret_cast<const uint4*>(src + 3 * P_ROW_BYTES);
                const uint2 xv = *reinterpret_cast<const uint2*>(xs + jrow);
                const uint32_t bac0 = is_b ? ((xv.x & 0xffffu) << bshift) : 0u;
                const uint32_t bbd0 = is_b ? ((xv.x >> 16) << bshift) : 0u;
                const uint32_t bac1 = is_b ? ((xv.y & 0xffffu) << bshift) : 0u;
                const uint32_t bbd1 = is_b ? ((xv.y >> 16) << bshift) : 0u;
                DqConst ka = ku, kb = ku, kc = ku, kd = ku;
                if (!UNIFORM) {
                    const uint2 gv = *reinterpret_cast<const uint2*>(sm.gidx + jrow);
                    int g0 = ibk + (int)(gv.x & 0xffffu), g1 = ibk + (int)(gv.x >> 16);
                    int g2 = ibk + (int)(gv.y & 0xffffu), g3 = ibk + (int)(gv.y >> 16);
                    g0 -= g0 >= op.Kb ? op.Kb : 0; g1 -= g1 >= op.Kb ? op.Kb : 0;
                    g2 -= g2 >= op.Kb ? op.Kb : 0; g3 -= g3 >= op.Kb ? op.Kb : 0;
                    if (op.Kb > op.n_alloc) { g0 %= op.n_alloc; g1 %= op.n_alloc; g2 %= op.n_alloc; g3 %= op.n_alloc; }
                    uint4 t;
                    t = sm.gtab[g0]; ka = {t.x, t.y, t.z};
                    t = sm.gtab[g1]; kb = {t.x, t.y, t.z};
                    t = sm.gtab[g2]; kc = {t.x, t.y, t.z};
                    t = sm.gtab[g3]; kd = {t.x, t.y, t.z};
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
            prefetch_next(pf, p, sm);   // refill the slot just consumed with this warp's unit 32 units ahead
        }

        trace_event(p, o, 3);
        // ---- flush the tile: cross-warp reduction in a fixed order ------------------------------
        // red[warp][lane][32 floats], 16-byte chunks rotated by the lane index (conflict-free 128-bit
        // accesses).  Every warp stores its sums; after one barrier every thread adds the 16 slots of its pair.
        {
            float4* mine = reinterpret_cast<float4*>(sm.red) + warp * (P_TI / 4) + lane * 8;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {   // outputs 4*ch .. 4*ch+3 of this lane's 32
                const int wd = ch >> 1, d0 = ch & 1;   // nibbles 4*d0 + {0,1,2,3} = (h0,d0) (h0,d0+2) (h1,d0) (h1,d0+2)
                mine[(ch + lane) & 7] = make_float4(acc[wd][0][d0], acc[wd][0][d0 + 2], acc[wd][1][d0], acc[wd][1][d0 + 2]);
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int d = 0; d < 4; ++d) acc[a][b][d] = 0.0f;
        }
        named_barrier(1, P_NCONS);
        float tot[2];
        {
            const int il = 2 * tid, ln = il >> 5, off = il & 31;
            const int fidx = ln * 32 + ((((off >> 2) + ln) & 7) << 2) + (off & 3);
            tot[0] = 0.0f;
            tot[1] = 0.0f;
#pragma unroll
            for (int sl = 0; sl < P_NCW; ++sl) {
                const float2 t2 = *reinterpret_cast<const float2*>(sm.red + sl * P_TI + fidx);
                tot[0] += t2.x;
                tot[1] += t2.y;
            }
        }
        if (k + seg < n_units) named_barrier(1, P_NCONS);   // another tile follows: its flush reuses the slots
        trace_event(p, o, 4);

        // ---- cross-CTA fix-up --------------------------------------------------------------------
        int cf, cl;
        tile_contributors(U, upt, op.n_tiles, tile, cf, cl);
        if (cf == cl) {
            epilogue(tile, tid, tot[0], tot[1], true);   // the tile is this CTA's alone
        } else {
            // Shared tile: every contributor stores its sums as (value, tag) words and moves on; the sums are
            // gathered after the unit loop, so that no CTA waits for another while it still owes partial sums.
            unsigned long long* slot = xchg_o + (size_t)(c + tile) * P_TI;
            st_relaxed_v2(slot + 2 * tid, pack_tagged(tot[0], tag), pack_tagged(tot[1], tag));
            if (n_shared == 0) sh_tile0 = tile;
            else sh_tile1 = tile;
            ++n_shared;
        }
        k += seg;
        r = 0;
        ++tile;
    }
    // ---- shared tiles: the outputs of a tile are dealt evenly to its contributors; each sums, in CTA order,
    // the tagged partial sums of all of them for its own outputs (a word is valid once it carries this
    // operator's tag: value and tag travel in one 64-bit store, so no flag, fence or second round trip)
    for (int sidx = 0; sidx < n_shared; ++sidx) {
        const int tile_s = sidx == 0 ? sh_tile0 : sh_tile1;
        int cf, cl, pp;
        tile_contributors(U, upt, op.n_tiles, tile_s, cf, cl);
        const bool active = slice_pair(cf, cl, c, tid, pp);
        const int n = cl - cf + 1, pb = pp - tid;
        const int cnt = (P_TI / 2) * (c - cf + 1) / n - pb, total = n * cnt;   // (contributor, pair) words to fetch
        // all threads fetch: word idx = contributor * cnt + pair, so that every load is in flight at once
        float2* stage = reinterpret_cast<float2*>(sm.xs);   // the input vector is no longer needed (unit loop is over)
        for (int base = 0; base < total; base += 2 * P_NCONS) {
            const int i0 = base + tid, i1 = i0 + P_NCONS;
            const bool h0 = i0 < total, h1 = i1 < total;
            const int c0 = i0 / cnt, c1 = i1 / cnt;
            const unsigned long long* s0p = xchg_o + (size_t)(cf + c0 + tile_s) * P_TI + 2 * (pb + i0 - c0 * cnt);
            const unsigned long long* s1p = xchg_o + (size_t)(cf + c1 + tile_s) * P_TI + 2 * (pb + i1 - c1 * cnt);
            unsigned long long a0 = 0, b0 = 0, a1 = 0, b1 = 0;
            const long long t_begin = clock64();
            for (;;) {
                if (h0) ld_relaxed_v2(s0p, a0, b0);
                if (h1) ld_relaxed_v2(s1p, a1, b1);
                const bool ok0 = !h0 || ((uint32_t)(a0 >> 32) == tag && (uint32_t)(b0 >> 32) == tag);
                const bool ok1 = !h1 || ((uint32_t)(a1 >> 32) == tag && (uint32_t)(b1 >> 32) == tag);
                if ((ok0 && ok1) || *sm.s_dead != 0) break;
                if (clock64() - t_begin > (1ll << 31)) {
                    atomicCAS(p.ws.err, 0, 0x50000 | o);   // a contributor's partial sums never arrived
                    *sm.s_dead = 1;
                    break;
                }
            }
            if (h0) stage[i0] = make_float2(__uint_as_float((uint32_t)a0), __uint_as_float((uint32_t)b0));
            if (h1) stage[i1] = make_float2(__uint_as_float((uint32_t)a1), __uint_as_float((uint32_t)b1));
        }
        named_barrier(1, P_NCONS);
        float s0 = 0.0f, s1 = 0.0f;
        if (active) {
            for (int cc = 0; cc < n; ++cc) {   // CTA order
                const float2 v = stage[cc * cnt + tid];
                s0 += v.x;
                s1 += v.y;
            }
        }
        trace_event(p, o, 5);
        epilogue(tile_s, pp, s0, s1, active);
        named_barrier(1, P_NCONS);   // stage is reused by the next shared tile
    }
    if (n_shared == 0) named_barrier(1, P_NCONS);   // every operator ends with a CTA barrier (see the operator loop)
    trace_event(p, o, 6);
    if (op.flags & PASS_PUBLISH) publish(p, o);   // this CTA's outputs of the operator are written
    trace_event(p, o, 7);
    if (op.epilogue == QW3_EPI_ARGMAX && c == 0 && warp == 0) {
        // whole-vocabulary winner (lowest index among equal maxima): CTA 0 waits for every CTA and reduces the
        // winners of all (CTA, tile) slices
        if (lane == 0 && *sm.s_dead == 0) {
            const long long t_begin = clock64();
            while (ld_acquire(p.done + o) < (int)gridDim.x) {
                if (clock64() - t_begin > (1ll << 31)) {
                    atomicCAS(p.ws.err, 0, 0x60000 | o);
                    *sm.s_dead = 1;
                    break;
                }
            }
        }
        __syncwarp();
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int t = lane; t < op.n_tiles; t += 32) {
            int cf, cl;
            tile_contributors(U, upt, op.n_tiles, t, cf, cl);
            for (int cc = cf; cc <= cl; ++cc) {
                const float ov = __ldcg(p.ws.arg_val + cc + t);
                const int oi = __ldcg(p.ws.arg_idx + cc + t);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0 && p.d_token_out) *p.d_token_out = bi;
        if (lane == 0 && p.tok_out_slot != nullptr) {
            // The first stage's next pass (position pos + 1) polls this word instead of waiting for a hand-off launch.
            unsigned long long* const dst = *p.tok_out_slot;
            const int gen = p.d_gen != nullptr ? __ldcg(p.d_gen) : 0;
            if (dst != nullptr && *sm.s_dead == 0)
                st_relaxed_sys_u64(dst, ((unsigned long long)peer_tag(gen, pos + 1) << 32) | (uint32_t)bi);
        }
    }
    uc_base += n_units;
}

// Eight halves that the operator before wrote as four tagged words: polled until all four carry its tag.
__device__ __forceinline__ uint4 load8_tagged(const PassParams& p, const PassSmem& sm, const unsigned long long* src,
                                              const uint32_t tag, const int code) {
    unsigned long long w0 = 0, w1 = 0, w2 = 0, w3 = 0;
    const long long t_begin = clock64();
    for (;;) {
        ld_relaxed_v2(src, w0, w1);
        ld_relaxed_v2(src + 2, w2, w3);
        if (((uint32_t)(w0 >> 32) == tag && (uint32_t)(w1 >> 32) == tag && (uint32_t)(w2 >> 32) == tag && (uint32_t)(w3 >> 32) == tag) ||
            *sm.s_dead != 0)
            break;
        if (clock64() - t_begin > (1ll << 31)) {
            atomicCAS(p.ws.err, 0, code);
            *sm.s_dead = 1;
            break;
        }
    }
    return make_uint4((uint32_t)w0, (uint32_t)w1, (uint32_t)w2, (uint32_t)w3);
}

// ---------------------------------------------------------------------------------------------
// Decode attention of one layer (attentionKernel, Inference.cu:182-266, intended math): work items
// (head, split of the KV length) are dealt round-robin to the CTAs; 32 half-warps of a CTA keep an
// online-softmax state each; the last CTA of a head merges its splits in a fixed order.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void att_merge_states(const float* st, int n, int i, float& M, float& L, float& O) {
    M = -INFINITY;
    for (int g = 0; g < n; ++g) M = fmaxf(M, st[g * WS_ATT_STRIDE + 128]);
    L = 0.0f;
    O = 0.0f;
    for (int g = 0; g < n; ++g) {
        const float m = st[g * WS_ATT_STRIDE + 128];
        const float w = (m == -INFINITY) ? 0.0f : expf(m - M);
        L += st[g * WS_ATT_STRIDE + 129] * w;
        O += st[g * WS_ATT_STRIDE + i] * w;
    }
}

__device__ __forceinline__ void attn_phase(const PassParams& p, const PassOpBody& op, const int o, const PassSmem& sm, const int pos) {
    const int tid = threadIdx.x, grp = tid >> 4, sl = tid & 15;
    const int G = gridDim.x, c = blockIdx.x, heads = p.heads;
    int S = G / heads;   // one (head, split) item per CTA
    S = S < 1 ? 1 : (S > WS_ATT_MAX_SPLITS ? WS_ATT_MAX_SPLITS : S);
    const int len = pos + 1;
    const int chunk = (len + S - 1) / S;
    const float scale = 1.0f / sqrtf(128.0f);
    float* st = sm.red;
    constexpr int NG = P_NCONS / 16;   // 32 half-warps
    unsigned long long* const xchg_o = p.xchg + (size_t)(o & 1) * P_PSLOTS * P_TI;
    const uint32_t xtag = (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)op.src;
    for (int item = c; item < heads * S; item += G) {
        const int head = item / S, split = item - head * S;
        const int p0 = split * chunk, p1 = min(len, p0 + chunk);
        const __half* kh = op.kc + (size_t)head * p.max_pos * 128 + sl * 8;
        const __half* vh = op.vc + (size_t)head * p.max_pos * 128 + sl * 8;
        constexpr int UN = 2;
        // Cache rows of earlier tokens do not depend on this token: the first batch is requested before q is
        // polled, and every later batch while the one before is being used.
        uint4 nk[UN], nv[UN];
        auto request_rows = [&](const int kb) {
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int kp = kb + grp + u * NG;
                nk[u] = make_uint4(0u, 0u, 0u, 0u);
                nv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (kp < p1 && !(kp == pos && op.xt != nullptr)) {
                    nk[u] = __ldcg(reinterpret_cast<const uint4*>(kh + (size_t)kp * 128));
                    nv[u] = __ldcg(reinterpret_cast<const uint4*>(vh + (size_t)kp * 128));
                }
            }
        };
        request_rows(p0);
        float qf[8];
        {
            const uint4 qv = op.xt != nullptr ? load8_tagged(p, sm, op.xt + head * 64 + sl * 4, xtag, 0x70000 | o)
                                              : __ldcg(reinterpret_cast<const uint4*>(op.x + head * 128 + sl * 8));
            const __half2* h = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                qf[2 * e] = f.x;
                qf[2 * e + 1] = f.y;
            }
        }
        trace_event(p, o, 2);
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
                if (kp < p1 && kp == pos && op.xt != nullptr) {
                    // this token's own row: the projection before wrote it to the cache for later tokens and as
                    // tagged words (behind q: k at hidden/2 words, v at hidden words) for this launch
                    kv[u] = load8_tagged(p, sm, op.xt + (p.hidden >> 1) + head * 64 + sl * 4, xtag, 0x70000 | o);
                    vv[u] = load8_tagged(p, sm, op.xt + p.hidden + head * 64 + sl * 4, xtag, 0x70000 | o);
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
        trace_event(p, o, 3);
#pragma unroll
        for (int e = 0; e < 8; ++e) st[grp * WS_ATT_STRIDE + sl * 8 + e] = ov[e];
        if (sl == 0) {
            st[grp * WS_ATT_STRIDE + 128] = m;
            st[grp * WS_ATT_STRIDE + 129] = l;
        }
        named_barrier(1, P_NCONS);
        // merge of the 32 half-warp states, same arithmetic and order as att_merge_states, but the weight
        // exp(m_g - M) of a state is computed once (lane g of warp 0) instead of once per output element
        float* wts = st + NG * WS_ATT_STRIDE;   // [NG] weights, then the maximum
        static_assert(NG == 32, "one lane per half-warp state");
        if (tid < 32) {
            const float mg = st[tid * WS_ATT_STRIDE + 128];
            float mx = mg;
#pragma unroll
            for (int msk = 16; msk > 0; msk >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, msk));
            wts[tid] = (mg == -INFINITY) ? 0.0f : expf(mg - mx);
            if (tid == 0) wts[NG] = mx;
        }
        named_barrier(1, P_NCONS);
        float M = 0.f, L = 1.f, O = 0.f;
        if (tid < 128) {
            M = wts[NG];
            L = 0.0f;
            O = 0.0f;
#pragma unroll 8
            for (int g = 0; g < NG; ++g) {
                const float w = wts[g];
                L += st[g * WS_ATT_STRIDE + 129] * w;
                O += st[g * WS_ATT_STRIDE + tid] * w;
            }
        }
        trace_event(p, o, 4);
        bool finalise = true;
        if (S > 1) {
            // split 0 of the head finalises; the other splits hand over their state (128 outputs, max, sum) as
            // tagged words, which split 0 polls: no flag, fence or second round trip
            const uint32_t tag = (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)o;
            if (split != 0) {
                unsigned long long* mine = xchg_o + (size_t)item * P_TI;
                if (tid < 128) st_relaxed_u64(mine + tid, pack_tagged(O, tag));
                if (tid == 0) {   // M and L are the same in all threads below 128
                    st_relaxed_u64(mine + 128, pack_tagged(M, tag));
                    st_relaxed_u64(mine + 129, pack_tagged(L, tag));
                }
                finalise = false;
            } else {
                named_barrier(1, P_NCONS);   // everybody has read st
                if (tid < 128) st[tid] = O;  // own state becomes row 0 of the merge table
                if (tid == 0) {
                    st[128] = M;
                    st[129] = L;
                }
                if (tid < 130) {
                    for (int sp = 1; sp < S; ++sp) {
                        const unsigned long long* src = xchg_o + (size_t)(item + sp) * P_TI + tid;
                        unsigned long long w;
                        const long long t_begin = clock64();
                        for (;;) {
                            w = ld_relaxed_u64(src);
                            if ((uint32_t)(w >> 32) == tag || *sm.s_dead != 0) break;
                            if (clock64() - t_begin > (1ll << 31)) {
                                atomicCAS(p.ws.err, 0, 0x70000 | o);   // a split's state never arrived
                                *sm.s_dead = 1;
                                break;
                            }
                        }
                        st[sp * WS_ATT_STRIDE + tid] = __uint_as_float((uint32_t)w);
                    }
                }
                named_barrier(1, P_NCONS);
                if (tid < 128) att_merge_states(st, S, tid, M, L, O);
            }
        }
        trace_event(p, o, 5);
        if (finalise && tid < 128) {   // four full warps: even lanes store the pair (plain and tagged)
            const __half v = __float2half_rn(O / L);
            const uint32_t mine = __half_as_ushort(v), next = __shfl_down_sync(0xffffffffu, mine, 1);
            if ((tid & 1) == 0) {
                const uint32_t pair = mine | (next << 16);
                const int i = head * 128 + tid;
                *reinterpret_cast<uint32_t*>(op.y + i) = pair;
                if (op.yt != nullptr) {
                    const uint32_t tag = (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)o;
                    st_relaxed_u64(op.yt + (i >> 1), ((unsigned long long)tag << 32) | pair);
                }
            }
        }
        trace_event(p, o, 6);
        named_barrier(1, P_NCONS);   // st is reused by the next item
    }
    if (c >= heads * S) named_barrier(1, P_NCONS);   // CTAs without an item: every operator ends with a CTA barrier
    if (op.flags & PASS_PUBLISH) publish(p, o);
}

// Embedding gather straight from the packed [hidden][vocab] matrix (Inference.cu:1310-1315).
__device__ __forceinline__ void embed_phase(const PassParams& p, const PassOpBody& op, const int o, const PassSmem& sm,
                                            const int pos) {
    const int tid = threadIdx.x, c = blockIdx.x;
    const int i = 2 * (c * P_NCONS + tid);   // this thread's pair of hidden elements
    const bool skip = p.d_skip != nullptr && __ldcg(p.d_skip) != 0;
    if (i < p.hidden) {
        uint32_t pair;
        if (skip) {
            pair = __ldcg(reinterpret_cast<const uint32_t*>(op.y + i));   // keep the hidden state of the pass before
        } else {
            long long tok;
            if (p.decode && (op.flags & PASS_TOKEN_PEER)) {
                // the id sampled by the last stage's pass of the previous position, stored from its GPU
                unsigned long long w = ld_relaxed_sys_u64(p.tok_in);
                const long long t_begin = clock64();
                while ((uint32_t)(w >> 32) != *sm.s_ptag && *sm.s_dead == 0) {
                    if (clock64() - t_begin > P_PEER_WAIT_CLOCKS) {
                        atomicCAS(p.ws.err, 0, 0xA0000 | o);   // the sampled id never arrived
                        *sm.s_dead = 1;
                        break;
                    }
                    w = ld_relaxed_sys_u64(p.tok_in);
                }
                tok = (long long)(int)(uint32_t)w;
            } else {
                tok = p.decode ? __ldcg(p.d_token) : __ldcg(p.d_prompt + pos);
            }
            if (tok < 0 || tok >= p.vocab) tok = 0;
            const long long pc = (p.vocab + 1) / 2;
            const long long g = (tok / 128) % op.n_alloc;
            const __half z = op.zp[g], sc = op.scale[g];
            uint32_t h[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t byte = op.packed[(long long)(i + e) * pc + (tok >> 1)];
                const uint32_t q = (tok & 1) ? (byte >> 4) : (byte & 15u);
                h[e] = __half_as_ushort(dequant_one(q, z, sc));
            }
            pair = h[0] | (h[1] << 16);
            *reinterpret_cast<uint32_t*>(op.y + i) = pair;
        }
        if (op.yt != nullptr) {
            const uint32_t tag = (uint32_t)*sm.s_epoch * (uint32_t)P_TAG_OPS + (uint32_t)o;
            st_relaxed_u64(op.yt + (i >> 1), ((unsigned long long)tag << 32) | pair);
        }
    }
    named_barrier(1, P_NCONS);   // every operator ends with a CTA barrier
    if (op.flags & PASS_PUBLISH) publish(p, o);
}

__global__ void __launch_bounds__(P_NTHREADS, 1) decode_pass_kernel(const PassParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    PassSmem sm;
    sm.ring = smem;
    sm.red = reinterpret_cast<float*>(smem + P_OFF_RED);
    sm.xs = reinterpret_cast<__half*>(smem + P_OFF_XS);
    sm.gidx = reinterpret_cast<uint16_t*>(smem + P_OFF_GIDX);
    sm.gtab = reinterpret_cast<uint4*>(smem + P_OFF_GTAB);
    uint8_t* misc = smem + P_OFF_MISC;
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc);              // full[P_RING]: 256 bytes
    sm.full0 = smem_u32(bars);
    sm.dsum = reinterpret_cast<double*>(misc + 640);                 // 128
    sm.s_argv = reinterpret_cast<float*>(misc + 768);                // 64
    sm.s_argi = reinterpret_cast<int*>(misc + 832);                  // 64
    sm.s_dead = reinterpret_cast<int*>(misc + 900);
    sm.s_epoch = reinterpret_cast<int*>(misc + 904);
    sm.s_ptag = reinterpret_cast<uint32_t*>(misc + 908);
    sm.s_op = reinterpret_cast<uint32_t*>(misc + 1024);              // 2 x 192 bytes

    const int tid = threadIdx.x, warp = tid >> 5;
    {   // this CTA's share of every operator, computed once (the prefetch cursors walk this table)
        int4* rng = reinterpret_cast<int4*>(smem + P_OFF_RNG);
        for (int o = tid; o < p.n_ops; o += P_NTHREADS) {
            const PassOpBody& b = p.ops[o].b;
            int ub = 0, n = 0;
            if (b.kind == PASS_GEMV) cta_range(b.U, b.upt, b.n_tiles, blockIdx.x, ub, n);
            rng[o] = make_int4(ub, n, b.upt, b.kind);
        }
        sm.s_rng = rng;
    }
    if (tid == 0) {
        for (int s = 0; s < P_RING; ++s) mbar_init(sm.full0 + 8 * s, 1);
        *sm.s_dead = 0;
        *sm.s_epoch = __ldcg(p.d_epoch) + 1;
        *sm.s_ptag = peer_tag(p.d_gen != nullptr ? __ldcg(p.d_gen) : 0, __ldcg(p.d_pos));
        mbar_fence_init();
    }
    __syncthreads();

    // prime the ring: the first two units of this warp (weights do not depend on activations)
    Prefetch pf;
    pf.op = -1; pf.uc = warp - P_NCW; pf.base = 0; pf.n = 0; pf.ub = 0; pf.upt = 1; pf.next_u = 0; pf.tile = 0; pf.r = 0; pf.end = false; pf.policy = l2_policy_evict_first();
    prefetch_next(pf, p, sm);
    prefetch_next(pf, p, sm);

    // ---------------- consumers ----------------------------------------------------------------
    const int pos = __ldcg(p.d_pos);
    if (tid < P_OPW) sm.s_op[tid] = reinterpret_cast<const uint32_t*>(&p.ops[0].b)[tid];
    int uc_base = 0;
    named_barrier(1, P_NCONS);   // descriptor of operator 0
    for (int o = 0; o < p.n_ops; ++o) {
        // Every operator ends with a CTA barrier after its last use of shared memory: the descriptor of this
        // operator (copied during the one before) is visible, and the buffer of the one before is free.
        trace_event(p, o, 0);
#ifdef QW3_TRACE
        if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            p.trace[o] = t;
        }
#endif
        const PassOpBody& op = *reinterpret_cast<const PassOpBody*>(sm.s_op + (o & 1) * P_OPW);
        if (o + 1 < p.n_ops && tid < P_OPW)   // next descriptor, visible after the barriers of this operator
            sm.s_op[((o + 1) & 1) * P_OPW + tid] = reinterpret_cast<const uint32_t*>(&p.ops[o + 1].b)[tid];
        if (op.kind == PASS_GEMV) {
            if (op.uniform) {
                if (op.exact) gemv_phase<true, true>(p, op, o, sm, uc_base, pos, pf);
                else gemv_phase<true, false>(p, op, o, sm, uc_base, pos, pf);
            } else {
                if (op.exact) gemv_phase<false, true>(p, op, o, sm, uc_base, pos, pf);
                else gemv_phase<false, false>(p, op, o, sm, uc_base, pos, pf);
            }
        } else if (op.kind == PASS_ATTN) {
            if (op.flags & PASS_WAIT_PREV) wait_for_previous(p, sm, o);
            attn_phase(p, op, o, sm, pos);
        } else {
            if (op.flags & PASS_WAIT_PREV) wait_for_previous(p, sm, o);
            embed_phase(p, op, o, sm, pos);
        }
    }
#ifdef QW3_TRACE
    if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[p.n_ops] = t;
    }
#endif
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
int encode_2d_u32(CUtensorMap* map, const void* base, uint64_t inner_elems, uint64_t rows, uint64_t pitch_bytes,
                  uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz);

int pass_init_device() {
    QW3_CUDA(cudaFuncSetAttribute(decode_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM_BYTES));
    int nb = 0;
    QW3_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, decode_pass_kernel, P_NTHREADS, P_SMEM_BYTES));
    if (nb < 1) {
        set_last_error("decode_pass_kernel does not fit on an SM (%zu bytes of shared memory)", P_SMEM_BYTES);
        return QW3_ERR_CUDA;
    }
    return QW3_OK;
}

// Whether a matrix can be an operator of the persistent pass (else the per-operator path is used).
bool pass_supports(const W4Desc* d) {
    if (d->K > P_MAXK || d->M > (long long)P_DONE * P_TI) return false;
    if (!d->uniform) {
        const long long Kb = d->K / 128, used = Kb < d->n_alloc ? Kb : d->n_alloc;
        if (d->K > P_MAXK_NU || used > P_MAX_GROUPS) return false;
    }
    return true;
}

void pass_fill_gemv(PassOp* op, const W4Desc* d, const void* x, const void* gamma, float eps, int epilogue, void* y,
                    void* kc, void* vc) {
    std::memset(op, 0, sizeof(*op));
    op->tmap = d->tmap;
    PassOpBody& b = op->b;
    b.kind = PASS_GEMV;
    b.uniform = d->uniform; b.exact = d->zp_integral; b.epilogue = epilogue;
    b.M = (int)d->M; b.K = (int)d->K; b.Mb = b.M / 128; b.Kb = b.K / 128;
    b.n_alloc = (int)d->n_alloc;
    b.n_tiles = (b.M + P_TI - 1) / P_TI;
    b.upt = b.K / P_UNIT_ROWS;
    b.U = (long long)b.n_tiles * b.upt;
    b.scale = d->scale; b.zp = d->zp;
    b.x = static_cast<const __half*>(x); b.gamma = static_cast<const __half*>(gamma);
    b.y = static_cast<__half*>(y); b.kc = static_cast<__half*>(kc); b.vc = static_cast<__half*>(vc);
    b.eps = eps;
}

void pass_fill_attn(PassOp* op, const void* q, void* kc, void* vc, void* ctx, int heads) {
    std::memset(op, 0, sizeof(*op));
    PassOpBody& b = op->b;
    b.kind = PASS_ATTN;
    b.x = static_cast<const __half*>(q);
    b.kc = static_cast<__half*>(kc); b.vc = static_cast<__half*>(vc);
    b.y = static_cast<__half*>(ctx);
}

void pass_fill_embed(PassOp* op, const void* packed, const void* scale, const void* zp, long long n_alloc, void* hidden_out,
                     int hidden) {
    std::memset(op, 0, sizeof(*op));
    PassOpBody& b = op->b;
    b.kind = PASS_EMBED;
    b.packed = static_cast<const uint8_t*>(packed);
    b.scale = static_cast<const __half*>(scale); b.zp = static_cast<const __half*>(zp);
    b.n_alloc = (int)n_alloc;
    b.y = static_cast<__half*>(hidden_out);
}

// How an operator is tied to its neighbours inside one launch: `xt` (written by operator `src`) replaces the
// plain input, `yt` receives a tagged copy of the output, `rt` (written by operator `rsrc`) holds the value a
// RESIDUAL epilogue adds to.
void pass_link(PassOp* op, int flags, int src, const void* xt, void* yt, const void* rt, int rsrc) {
    op->b.flags = flags;
    op->b.src = src;
    op->b.rsrc = rsrc;
    op->b.xt = static_cast<const unsigned long long*>(xt);
    op->b.yt = static_cast<unsigned long long*>(yt);
    op->b.rt = static_cast<const unsigned long long*>(rt);
}

size_t pass_op_bytes() { return sizeof(PassOp); }
// Exchange buffer of tagged partial sums: one 1024-word slot per (CTA, tile) pair c + tile.
size_t pass_xchg_bytes() { return 2 * (size_t)P_PSLOTS * P_TI * sizeof(unsigned long long); }

// Enqueues one pass: clears the arrival counters, then one cooperative launch.  The caller increments
// *d_epoch on the same stream afterwards.
int pass_launch(const void* d_ops, int n_ops, int* d_done, unsigned long long* d_xchg, const int* d_epoch, const int* d_pos, const int* d_token, const int* d_skip,
                const int* d_prompt, int decode, const void* cos_t, const void* sin_t, int heads, int hidden,
                long long max_pos, long long vocab, int* d_token_out, float* logits_f32, unsigned long long* trace,
                unsigned long long* trace2, const int* d_gen, const void* tok_in, const void* tok_out_slot, const Workspace* ws,
                cudaStream_t st) {
    QW3_REQUIRE(n_ops <= P_MAX_OPS, "pass_launch: too many operators in one pass");
    PassParams p;
    std::memset(&p, 0, sizeof(p));
    p.ops = static_cast<const PassOp*>(d_ops);
    p.n_ops = n_ops;
    p.done = d_done;
    p.xchg = d_xchg;
    p.d_epoch = d_epoch;
    p.d_pos = d_pos; p.d_token = d_token; p.d_skip = d_skip; p.d_prompt = d_prompt;
    p.decode = decode;
    p.cos_t = static_cast<const __half*>(cos_t); p.sin_t = static_cast<const __half*>(sin_t);
    p.heads = heads; p.hidden = hidden; p.max_pos = max_pos; p.vocab = vocab;
    p.d_token_out = d_token_out; p.logits_f32 = logits_f32; p.trace = trace; p.trace2 = trace2;
    p.d_gen = d_gen;
    p.tok_in = static_cast<const unsigned long long*>(tok_in);
    p.tok_out_slot = static_cast<unsigned long long* const*>(tok_out_slot);
    p.ws = *ws;
    int grid = ws->sm_count < WS_MAX_CTAS ? ws->sm_count : WS_MAX_CTAS;
    QW3_CUDA(cudaMemsetAsync(d_done, 0, (size_t)n_ops * sizeof(int), st));
    void* args[] = {&p};
    QW3_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(decode_pass_kernel), dim3(grid), dim3(P_NTHREADS), args,
                                         P_SMEM_BYTES, st));
    return QW3_OK;
}

}  // namespace qw3
