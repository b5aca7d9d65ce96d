// Exchange of row blocks between the GPUs of one node through peer-mapped memory, for the key / value all-gather of a
// global attention layer whose frames are sharded over the GPUs (one process per GPU).
//
// Every rank owns one "window": a cudaMalloc'ed buffer that the other ranks map through a CUDA IPC handle.  A rank puts
// its block into its own window (a local copy), tells the others with one release store per peer into THEIR flag words
// (peer_signal_kernel), waits until every peer has told it the same (peer_wait_kernel, bounded), and then PULLS the
// peers' blocks with plain cudaMemcpyAsync calls: the driver moves the bytes over NVLink without any kernel of this library,
// so a persistent attention kernel on the same GPU keeps all but the two SMs of the two small kernels; the rows land in
// this GPU's own memory, where the attention kernel reads them with its ordinary TMA loads.  No multicast, no kernel that
// takes a peer pointer as a tensor operand: the only peer accesses of a kernel are the flag stores.
//
// The wait is bounded (a time limit in nanoseconds of %globaltimer): when it runs out the kernel raises bit 18 of the
// library's device status word and returns; nothing hangs, and the caller finds the word raised.
#include "come_internal.cuh"

#include <cstring>

namespace come {

namespace {

constexpr unsigned int kErrPeerWait = 1u << 18;
constexpr int kMaxPeers = 64;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Thread p tells rank p: "rank `rank` has reached `value`" (flag word `rank` of p's flag array).
__global__ void peer_signal_kernel(int32_t *const *__restrict__ peer_flags, int world, int rank, int32_t value) {
    const int p = threadIdx.x;
    if (p < world && p != rank) {
        int32_t *dst = peer_flags[p] + rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(value) : "memory");
    }
}

// Thread p waits until rank p has reached `value` (this rank's own flag word p, written by rank p).
__global__ void peer_wait_kernel(const int32_t *__restrict__ flags, int world, int rank, int32_t value, long long limit_ns,
                                 unsigned int *__restrict__ status) {
    const int p = threadIdx.x;
    if (p >= world || p == rank) return;
    const unsigned long long t0 = global_ns();
    while (true) {
        int32_t v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + p) : "memory");
        if ((int32_t)(v - value) >= 0) return;  // wrap-around safe "v >= value"
        if ((long long)(global_ns() - t0) > limit_ns) {
            atomicOr(status, kErrPeerWait);
            return;
        }
        __nanosleep(256);
    }
}

}  // namespace

}  // namespace come

using namespace come;

extern "C" int come_peer_alloc(int64_t bytes, void **ptr_out, void *handle_out) {
    COME_REQUIRE(bytes > 0 && ptr_out && handle_out, "bytes must be > 0, ptr_out and handle_out not NULL");
    void *p = nullptr;
    COME_CUDA(cudaMalloc(&p, (size_t)bytes));
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        set_error("come_peer_alloc: %s", cudaGetErrorString(e));
        cudaFree(p);
        return COME_ERR_CUDA;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == COME_PEER_HANDLE_BYTES, "IPC handle size");
    std::memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return COME_OK;
}

extern "C" int come_peer_open(const void *handle, void **ptr_out) {
    COME_REQUIRE(handle && ptr_out, "handle and ptr_out must not be NULL");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    COME_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return COME_OK;
}

extern "C" int come_peer_close(void *ptr) {
    if (ptr) COME_CUDA(cudaIpcCloseMemHandle(ptr));
    return COME_OK;
}

extern "C" int come_peer_free(void *ptr) {
    if (ptr) COME_CUDA(cudaFree(ptr));
    return COME_OK;
}

extern "C" int come_peer_copy(void *dst, const void *src, int64_t bytes, void *stream) {
    COME_REQUIRE(bytes >= 0, "bytes must be >= 0");
    if (bytes == 0) return COME_OK;
    COME_REQUIRE(dst && src, "dst and src must not be NULL");
    COME_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    return COME_OK;
}

extern "C" int come_peer_signal(void *const *peer_flags_dev, int world, int rank, int32_t value, void *stream) {
    COME_REQUIRE(peer_flags_dev && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world,
                 "peer_flags must not be NULL, 1 <= world <= %d, 0 <= rank < world", kMaxPeers);
    if (world == 1) return COME_OK;
    peer_signal_kernel<<<1, kMaxPeers, 0, (cudaStream_t)stream>>>(reinterpret_cast<int32_t *const *>(peer_flags_dev), world, rank, value);
    return check_launch("come_peer_signal");
}

extern "C" int come_peer_wait(const int32_t *flags_dev, int world, int rank, int32_t value, int64_t limit_ns, void *stream) {
    COME_REQUIRE(flags_dev && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world,
                 "flags must not be NULL, 1 <= world <= %d, 0 <= rank < world", kMaxPeers);
    COME_REQUIRE(limit_ns > 0 && limit_ns <= 120ll * 1000 * 1000 * 1000, "limit_ns must be in (0, 120 s]");
    if (world == 1) return COME_OK;
    unsigned int *status = status_word_dev();
    if (!status) return COME_ERR_CUDA;
    peer_wait_kernel<<<1, kMaxPeers, 0, (cudaStream_t)stream>>>(flags_dev, world, rank, value, (long long)limit_ns, status);
    return check_launch("come_peer_wait");
}
