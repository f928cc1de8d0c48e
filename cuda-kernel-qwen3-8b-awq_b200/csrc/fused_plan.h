// Work split and weight-stream layout of the fused token pass (fused_pass.cu), shared by the kernel, the load-time
// repack and the host-side planner.
//
// The reference keeps every matrix as the flat nibble stream dequantAwqKernel reads (Inference.cu:84-105) and lets
// cuBLAS walk it column-major (Inference.cu:1052-1065).  The on-disk files keep that layout (Inference.cu:780-900);
// at load time each matrix is additionally rewritten, on the device, into the order in which the fused pass consumes
// it: one byte stream per (CTA, warp), made of 512-byte items; the 16 warp streams of a CTA are interleaved in pieces of
// whole k-groups ([unit][warp][piece]) so that one bulk copy fetches the next piece of every warp.  An item is the A operand of two
// m16n8k32 integer MMAs: 16 outputs x 64 inputs, every lane owning one 16-byte piece = four 32-bit words, the eight
// nibbles of a word sitting where one AND per register turns them into the u8 A fragment.  (A trailing half group of
// 32 inputs makes a 256-byte item, one MMA.)
//
// A GEMV operator is cut twice.  Across CTAs: CTA c owns n_mt tiles of 16 outputs and n_ks k-steps of 16 inputs.
// Across the 16 warps of a CTA: wm = 16 / wk warps along the tiles, wk warps along the k-steps; warp (a, bk) walks its
// nb tile blocks of tb tiles each, and for every block its k-share in groups of four k-steps:
//     for block: for group: for tile in block: one item
// so the B fragment (the activations of a group) is loaded once per group and block, and the tb accumulators of a block
// stay in registers.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define QW3_HD __host__ __device__ __forceinline__
#else
#define QW3_HD inline
#endif

namespace qw3 {

constexpr int F_NW = 16;          // warps per CTA
#ifndef QW3_F_UNIT
#define QW3_F_UNIT 3072
#endif
constexpr int F_UNIT = QW3_F_UNIT;   // largest piece of one warp in a ring unit (a unit = 16 pieces = one bulk copy)

enum FusedOp { F_QKV = 0, F_WO = 1, F_W1 = 2, F_W2 = 3, F_UNEMB = 4, F_NOPS = 5 };

struct FGemvPlan {
    int n_cta;        // CTAs that take part (the others skip the operator)
    int n_mt;         // tiles of 16 outputs per CTA
    int n_ks;         // k-steps of 16 inputs per CTA
    int wk;           // warps along the k-steps (16 / wk along the tiles)
    int tb, nb;       // per warp: nb blocks of tb tiles
    int nq, rem;      // per warp: n_ks / wk = 4 * nq + rem, rem in {0, 2}
    int warp_bytes;   // bytes of one warp's stream = nb * tb * (nq * 512 + rem * 128)
    int gu;           // k-groups per ring unit (rem == 0; with a half group the whole block is one unit)
    int unit_bytes;   // bytes of one warp's piece of a unit: gu * tb * 512, or the block's tb * (nq * 512 + rem * 128)
    int n_units;      // ring units of one warp's stream = warp_bytes / unit_bytes
};

// Geometry every rank and CTA derives its slices from.
struct FusedGeom {
    int H, I, heads, vocab;     // model
    int n_ranks, rank;          // row-split across GPUs (1, 0: one GPU holds every matrix whole)
    int heads_local;            // heads / n_ranks
    int gs;                     // CTAs that share one head (split of the Wqkv inputs, of the KV length, of the Wo outputs)
    int n_act;                  // CTAs that run the layers = heads_local * gs
    int rs;                     // hidden elements a CTA reduces and owns = H / (n_ranks * n_act)
    int n_mlp;                  // CTAs that run W1 / W2 (the first n_mlp of the n_act)
    int n1;                     // W1 outputs per such CTA = I / (n_ranks * n_mlp)
    int n_blocks;               // vocab / 128
    int grid;                   // CTAs launched (all of them take part in the unembedding)
};

// Position of one 32-bit word of a warp's stream.
struct FWordPos {
    int tile;      // tile index within the CTA: (a * nb + block) * tb + i
    int kstep;     // k-step within the CTA: bk * (4 nq + rem) + 4 * group (+ s)  -- first k-step of the group
    int gsteps;    // k-steps of the group: 4, or 2 for the trailing half group
    int lane, s;   // lane that loads the word and the k-step of the group it feeds
};

QW3_HD FWordPos fused_word_pos(const FGemvPlan& pl, int warp, int byte_off) {
    FWordPos r;
    const int a = warp / pl.wk, bk = warp % pl.wk;
    const int full = pl.nq * pl.tb * 512;
    const int block_bytes = full + pl.tb * pl.rem * 128;
    const int b = byte_off / block_bytes, ob = byte_off % block_bytes;
    int q, i, within;
    if (ob < full) {
        q = ob / (pl.tb * 512);
        i = (ob % (pl.tb * 512)) / 512;
        within = ob % 512;
        r.gsteps = 4;
        r.lane = within / 16;
        r.s = (within % 16) / 4;
    } else {
        const int o2 = ob - full;
        q = pl.nq;
        i = o2 / 256;
        within = o2 % 256;
        r.gsteps = 2;
        r.lane = within / 8;
        r.s = (within % 8) / 4;
    }
    r.tile = (a * pl.nb + b) * pl.tb + i;
    r.kstep = bk * (4 * pl.nq + pl.rem) + 4 * q;
    return r;
}

// Where byte `stream_off` of a CTA's interleaved stream belongs: which warp, and which byte of that warp's own stream.
// Unit u holds bytes [u * unit_bytes, (u + 1) * unit_bytes) of every warp's stream, warp after warp.
QW3_HD void fused_stream_locate(const FGemvPlan& pl, int stream_off, int& warp, int& warp_off) {
    const int u = stream_off / (F_NW * pl.unit_bytes), in_unit = stream_off % (F_NW * pl.unit_bytes);
    warp = in_unit / pl.unit_bytes;
    warp_off = u * pl.unit_bytes + in_unit % pl.unit_bytes;
}

// The eight nibbles of a word: nibble n (bits 4n .. 4n+3) holds W[row][j] with
//   row = g + 8 * (n & 1)            (g = lane / 4: the low nibble of every byte belongs to row g of the tile, the high one to row g + 8)
//   j   = 16 * kstep + 4 * gsteps * t + 4 * s + (n >> 1)                           (t = lane % 4)
// so that `w & 0x0f0f0f0f` and `w & 0xf0f0f0f0` of the words s = 0, 1 (and of s = 2, 3) of a lane are the u8 A fragment
// of mma.sync.m16n8k32 (a0: row g, bytes k 4t..4t+3; a1: row g + 8; a2, a3: the same for k + 16) when the B fragment
// of lane t holds, byte for byte, the inputs 16*kstep + 4*gsteps*t + 4*s + {0, 1, 2, 3}: lane t owns 4 * gsteps
// consecutive inputs of the group.  (The MMA sums over all 32 k positions of a fragment, so which input sits at which
// position is free as long as A and B agree.)
QW3_HD void fused_nibble_src(const FWordPos& w, int n, int& row, int& j) {
    const int g = w.lane >> 2, t = w.lane & 3;
    row = g + 8 * (n & 1);
    j = 16 * w.kstep + 4 * w.gsteps * t + 4 * w.s + (n >> 1);
}

// First output of tile `tile` of CTA `cta` (the tile covers 16 consecutive outputs), or -1 when the CTA has no such
// tile, and the first input of the CTA's k-steps.  `blk` is the 128-output block of an unembedding step.
QW3_HD long long fused_tile_out(const FusedGeom& g, int op, int cta, int tile, long long blk) {
    switch (op) {
        case F_QKV: {   // tiles 0-7: q of the CTA's head, 8-15: k, 16-23: v (Inference.cu:1070-1072: q | k | v sections)
            const int head = g.rank * g.heads_local + cta / g.gs;
            return (long long)(tile / 8) * g.H + head * 128 + (tile % 8) * 16;
        }
        case F_WO:      // the outputs are cut evenly among the gs CTAs of a head
            return (long long)(cta % g.gs) * (g.H / g.gs) + tile * 16;
        case F_W1:
            return (long long)(g.rank * g.n_mlp + cta) * g.n1 + tile * 16;
        case F_W2:
            return (long long)tile * 16;
        default:
            return blk * 128 + tile * 16;
    }
}
QW3_HD long long fused_k0(const FusedGeom& g, int op, int cta) {
    switch (op) {
        case F_QKV: return (long long)(cta % g.gs) * (g.H / g.gs);
        case F_WO:  return (long long)(g.rank * g.heads_local + cta / g.gs) * 128;
        case F_W2:  return (long long)(g.rank * g.n_mlp + cta) * g.n1;
        default:    return 0;
    }
}

// Block of 128 vocabulary entries that CTA `cta` handles in round `round` of the unembedding (-1: none).
QW3_HD long long fused_unemb_block(const FusedGeom& g, int cta, int round) {
    const long long b = ((long long)round * g.n_ranks + g.rank) * g.grid + cta;
    return b < g.n_blocks ? b : -1;
}

}  // namespace qw3
