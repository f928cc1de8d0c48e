// Host interface of the fused token pass (fused_pass.cu) towards the engine.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "fused_plan.h"

namespace qw3 {

struct FusedMatrix {           // one AWQ matrix as loaded from disk (AWQWeight without d_dq, Inference.cu:318-325)
    const void* packed;
    const void* scale;
    const void* zp;
    long long n_alloc, out_dim, in_dim;
};
struct FusedLayerIn {
    FusedMatrix m[4];          // Wqkv, Wo, W1, W2
    const void* gamma;
    void* kc;
    void* vc;
};
struct FusedCreate {
    int H, I, heads, vocab, n_layers;
    float eps;
    int attn_split_min;        // contexts longer than this are split over the CTAs of a head group
    int no_cluster;            // 1: head groups exchange through global memory even where a thread-block cluster could carry them
    long long max_pos;
    int n_ranks, rank;         // row-split over GPUs (1, 0 otherwise)
    int sm_count, device;
    const FusedLayerIn* layers;
    const FusedMatrix* emb;    // first stage (null elsewhere)
    const FusedMatrix* unemb;  // last stage (null elsewhere)
    const void* gamma_final;
    void* hidden;
    int *d_pos, *d_token, *d_skip, *d_prompt, *d_gen;
    const void *cos_t, *sin_t;
    void* logits16;
    float* logits32;
    int* err;
    cudaStream_t stream;
};

struct FusedPass;

// Whether (and how) the fused pass covers a configuration: geometry and the five operator plans.
bool fused_plan(int H, int I, int heads, int vocab, int n_layers, long long max_pos, int n_ranks, int rank, int grid,
                FusedGeom* geom, FGemvPlan* plans);
size_t fused_stream_bytes(const FusedGeom& g, const FGemvPlan& pl, int op);
// The load-time repack on the host (what fused_repack_kernel does on the device), for tests of the layout.
void fused_repack_host(const FusedGeom& g, const FGemvPlan& pl, int op, const uint8_t* raw, long long out_dim, uint8_t* out);

// Repacks the matrices of a stage on its device, allocates the exchange buffers, keeps the launch parameters.
int fused_create(const FusedCreate& a, FusedPass** out);
void fused_destroy(FusedPass* f);
// One token pass (decode != 0: with final norm, unembedding and arg-max when the stage has them).
int fused_launch(FusedPass* f, int decode, cudaStream_t st);
// Row-split over GPUs: this rank's exchange buffers (to export) and the peers' mappings of theirs.
void* fused_exchange_base(FusedPass* f, size_t* bytes);
void fused_set_peer(FusedPass* f, int rank, void* base);
void fused_geometry(const FusedPass* f, FusedGeom* g, FGemvPlan* plans);
const void* fused_trace(const FusedPass* f, size_t* bytes);

}  // namespace qw3
