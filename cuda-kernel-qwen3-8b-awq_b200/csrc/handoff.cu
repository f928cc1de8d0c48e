// Stage hand-off between GPUs for the one-process-per-GPU layer pipeline (sm_100a, NVLink P2P).
//
// The reference moves the hidden state between its two GPUs with cudaMemcpyPeerAsync from one host
// thread and a host synchronisation per copy (copyHiddenBetweenGPUs, Inference.cu:1013-1023,
// 1335-1336, 1357-1358).  With one process per GPU the stages are chained on the device instead:
// every stage owns a mailbox in its own memory; its ring neighbours map it through CUDA IPC and
//   * the sender stores the 8 KB hidden state straight into the receiver's inbox (plain peer
//     stores over NVLink), fences at system scope and releases the receiver's flag;
//   * the receiver's stream holds a one-CTA kernel that acquire-polls that flag (bounded: about
//     nine seconds, then it records an error and returns), copies the inbox out and acknowledges
//     into the sender's mailbox, which is what lets the sender reuse the two inbox slots;
//   * the sampled token id travels the same way from the last stage to the first.
// That protocol serves the prompt phase and the first decode step.  From the second decode step on the stages are
// chained inside the token-pass kernels (decode_pass.cu): the mailbox also holds a tagged inbox and a tagged token
// word which the kernels store to and poll directly, so no hand-off launch sits between two stages.
// No collective exists on this path, so no NCCL; no multicast of any kind is used.
#include "common.cuh"

namespace qw3 {

struct Mailbox {
    int in_flag;     // number of the newest hidden-state message delivered into `inbox`
    int ack_flag;    // number of the newest message the stage after this one has taken out of ITS inbox
    int tok_flag;    // number of the newest token message
    int tok_val;
    int blk_flag;    // number of the newest block of prompt rows delivered into `block_inbox`
    int blk_ack;     // number of the newest block the stage after this one has taken out of ITS block inbox
    int pad0[10];
    unsigned long long tok_word;   // byte 64: (sampled id, tag) stored by the last stage's token-pass kernel itself
    int pad1[46];
    // followed by __half inbox[2][hidden], then unsigned long long linked_inbox[hidden / 2]: the hidden state as
    // (two halves, tag) words stored by the last operator of the previous stage's token-pass kernel and polled by
    // the first operator of this stage's (decode steps chained inside the kernels, no hand-off launches),
    // then __half block_inbox[2][block_rows][hidden]: blocks of prompt rows of the batched prompt phase
};
static_assert(sizeof(Mailbox) == 256, "mailbox header is 256 bytes");

constexpr int MB_BLOCK_ROWS = 2048;  // largest block of prompt rows handed over at once (PF_BLOCK of the engine)
size_t mailbox_bytes(int hidden) {
    return sizeof(Mailbox) + (size_t)2 * hidden * 2 + (size_t)(hidden / 2) * 8 + (size_t)2 * MB_BLOCK_ROWS * hidden * 2;
}
void* mailbox_block_inbox(void* mb, int hidden, int slot) {
    return static_cast<uint8_t*>(mb) + sizeof(Mailbox) + (size_t)2 * hidden * 2 + (size_t)(hidden / 2) * 8 +
           (size_t)slot * MB_BLOCK_ROWS * hidden * 2;
}
void* mailbox_linked_inbox(void* mb, int hidden) { return static_cast<uint8_t*>(mb) + sizeof(Mailbox) + (size_t)2 * hidden * 2; }
void* mailbox_token_word(void* mb) { return &static_cast<Mailbox*>(mb)->tok_word; }

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *flag >= want.  Returns false after `limit` clocks (default ~2^34, about nine seconds).
constexpr long long HANDOFF_WAIT_CLOCKS = 1ll << 34;
__device__ __forceinline__ bool wait_flag(const int* flag, int want, long long limit = HANDOFF_WAIT_CLOCKS) {
    const long long t0 = clock64();
    while (ld_acquire_sys(flag) < want) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
    return true;
}

__global__ void __launch_bounds__(256) handoff_send_kernel(const __half* __restrict__ hidden, Mailbox* next_mb,
                                                           const Mailbox* my_mb, int msg, int n_chunks, int* err) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        s_ok = wait_flag(&my_mb->ack_flag, msg - 2) ? 1 : 0;   // slot msg&1 was last used by message msg-2
        if (!s_ok) atomicCAS(err, 0, 0x40001);
    }
    __syncthreads();
    if (!s_ok) return;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(next_mb) + sizeof(Mailbox)) + (size_t)(msg & 1) * n_chunks;
    const uint4* src = reinterpret_cast<const uint4*>(hidden);
    for (int i = threadIdx.x; i < n_chunks; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(&next_mb->in_flag, msg);
}

__global__ void __launch_bounds__(256) handoff_recv_kernel(__half* __restrict__ hidden, const Mailbox* my_mb, Mailbox* prev_mb,
                                                           int msg, int n_chunks, int* err) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        s_ok = wait_flag(&my_mb->in_flag, msg) ? 1 : 0;
        if (!s_ok) atomicCAS(err, 0, 0x40002);
    }
    __syncthreads();
    if (!s_ok) return;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(my_mb) + sizeof(Mailbox)) + (size_t)(msg & 1) * n_chunks;
    uint4* dst = reinterpret_cast<uint4*>(hidden);
    for (int i = threadIdx.x; i < n_chunks; i += blockDim.x) dst[i] = __ldcg(src + i);
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(&prev_mb->ack_flag, msg);
}

__global__ void token_send_kernel(const int* __restrict__ d_token, Mailbox* first_mb, int msg) {
    if (threadIdx.x != 0) return;
    first_mb->tok_val = *d_token;
    __threadfence_system();
    st_release_sys(&first_mb->tok_flag, msg);
}

__global__ void token_recv_kernel(int* __restrict__ d_token, const Mailbox* my_mb, int msg, int* err) {
    if (threadIdx.x != 0) return;
    if (!wait_flag(&my_mb->tok_flag, msg)) {
        atomicCAS(err, 0, 0x40003);
        return;
    }
    *d_token = __ldcg(&my_mb->tok_val);
}

// Blocks of prompt rows: the rows move with a copy-engine copy between the two GPUs; these two one-thread kernels
// around it carry the protocol (wait for the flag, bounded; publish the flag after the copy before it in the stream).
__global__ void flag_wait_kernel(const int* flag, int want, int* err, int code, long long limit) {
    if (threadIdx.x == 0 && !wait_flag(flag, want, limit)) atomicCAS(err, 0, code);
}
__global__ void flag_set_kernel(int* flag, int value) {
    if (threadIdx.x != 0) return;
    __threadfence_system();
    st_release_sys(flag, value);
}

// Block `msg` (1, 2, ...) of `bytes` from `rows_src` into the next stage's block inbox.
int block_send(const void* rows_src, size_t bytes, void* next_mb, const void* my_mb, int msg, int hidden, int* err, cudaStream_t st) {
    flag_wait_kernel<<<1, 32, 0, st>>>(&static_cast<const Mailbox*>(my_mb)->blk_ack, msg - 2, err, 0x40004, HANDOFF_WAIT_CLOCKS);
    QW3_CUDA(cudaGetLastError());
    QW3_CUDA(cudaMemcpyAsync(mailbox_block_inbox(next_mb, hidden, msg & 1), rows_src, bytes, cudaMemcpyDeviceToDevice, st));
    flag_set_kernel<<<1, 32, 0, st>>>(&static_cast<Mailbox*>(next_mb)->blk_flag, msg);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
// Block `msg` out of this stage's block inbox into `rows_dst`, then the acknowledgement to the stage before.
int block_recv(void* rows_dst, size_t bytes, void* my_mb, void* prev_mb, int msg, int hidden, int* err, cudaStream_t st) {
    flag_wait_kernel<<<1, 32, 0, st>>>(&static_cast<const Mailbox*>(my_mb)->blk_flag, msg, err, 0x40005, HANDOFF_WAIT_CLOCKS);
    QW3_CUDA(cudaGetLastError());
    QW3_CUDA(cudaMemcpyAsync(rows_dst, mailbox_block_inbox(my_mb, hidden, msg & 1), bytes, cudaMemcpyDeviceToDevice, st));
    flag_set_kernel<<<1, 32, 0, st>>>(&static_cast<Mailbox*>(prev_mb)->blk_ack, msg);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

int handoff_send(const void* hidden, void* next_mb, const void* my_mb, int msg, int hidden_n, int* err, cudaStream_t st) {
    handoff_send_kernel<<<1, 256, 0, st>>>(static_cast<const __half*>(hidden), static_cast<Mailbox*>(next_mb),
                                           static_cast<const Mailbox*>(my_mb), msg, hidden_n / 8, err);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int handoff_recv(void* hidden, const void* my_mb, void* prev_mb, int msg, int hidden_n, int* err, cudaStream_t st) {
    handoff_recv_kernel<<<1, 256, 0, st>>>(static_cast<__half*>(hidden), static_cast<const Mailbox*>(my_mb),
                                           static_cast<Mailbox*>(prev_mb), msg, hidden_n / 8, err);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int token_send(const int* d_token, void* first_mb, int msg, cudaStream_t st) {
    token_send_kernel<<<1, 32, 0, st>>>(d_token, static_cast<Mailbox*>(first_mb), msg);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}
int token_recv(int* d_token, const void* my_mb, int msg, int* err, cudaStream_t st) {
    token_recv_kernel<<<1, 32, 0, st>>>(d_token, static_cast<const Mailbox*>(my_mb), msg, err);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

// Test hook: the protocol's wait kernel on a flag of the caller with a caller-chosen limit, so that a wait can be made to
// run out in milliseconds (the flag is simply never set): the kernel returns, the error word carries `code`.
int flag_wait_launch(const int* d_flag, int want, long long limit_clocks, int* err, int code, cudaStream_t st) {
    flag_wait_kernel<<<1, 32, 0, st>>>(d_flag, want, err, code, limit_clocks);
    QW3_CUDA(cudaGetLastError());
    return QW3_OK;
}

}  // namespace qw3
