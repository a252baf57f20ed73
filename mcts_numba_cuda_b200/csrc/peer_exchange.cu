// Sum of small int64 vectors over the GPUs of one box without a collective library: every rank stores its vector
// into a slot of every peer's buffer (plain stores to peer memory over NVLink), raises a flag there, waits -- bounded --
// for the flags of all ranks in its own buffer and adds the slots up locally.  Remote data is only ever written, reads
// are local.  Plain stores and loads only.
//
// The exchange step of root-parallel search: per batch and rank 3 * max_actions int64 per search, a few tens of KB (the
// reference is single-GPU: its _reduce_over_trees_* sums over trees of one device, src/mctsnc.py:2223-2296; sharding the
// trees over GPUs puts this sum between it and _reduce_over_actions_*).  At this size a collective is pure latency;
// one store kernel and one add kernel on the caller's stream cost a few microseconds and need no second library.
//
// Protocol.  Call k (k = 1, 2, ...) uses half k % 2 of every buffer.  Writer: all data stores, __threadfence_system(),
// then flag[half][rank] = k in every peer's buffer.  Reader: waits until flag[half][r] >= k for every r, then reads the
// slots with loads that bypass L1.  A rank can start call k + 2 (same half) only after its call k + 1 has seen the flags
// of all ranks for k + 1, which every rank raises after finishing its call k: nobody overwrites a half that is still
// being read.  The wait gives up after `wait_limit` polls and sets the status word instead of hanging; the values are
// then left as they were.
#include "../../include/mctsnc_b200.h"

#include <cuda_runtime.h>

#include <new>

namespace {

constexpr int MAX_WORLD = 64;
constexpr int EXCHANGE_THREADS = 1024;

#define CUDA_TRY(expr)                        \
    do {                                      \
        cudaError_t _e = (expr);              \
        if (_e != cudaSuccess) return (int)_e; \
    } while (0)

struct PeerTable {
    long long *data[MAX_WORLD];   // peer r's buffer: [2][world][n_max] int64
    int *flags[MAX_WORLD];        // peer r's flags:  [2][world]
};

__global__ void __launch_bounds__(EXCHANGE_THREADS) push_kernel(PeerTable peers, const long long *values, long long n, long long n_max,
                                                                int rank, int world, int call) {
    const int half = call & 1;
    for (int p = 0; p < world; p++) {
        long long *dst = peers.data[p] + ((long long)half * world + rank) * n_max;
        for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = values[i];
    }
    __threadfence_system();   // this thread's stores are visible to the peers before the flag is
    __syncthreads();
    if (threadIdx.x < world) {
        __threadfence_system();
        *(volatile int *)(peers.flags[threadIdx.x] + half * world + rank) = call;
    }
}

__global__ void __launch_bounds__(EXCHANGE_THREADS) sum_kernel(const long long *data, const int *flags, long long *values, long long n,
                                                               long long n_max, int world, int call, int wait_limit, int *status) {
    __shared__ int s_missing;
    const int half = call & 1;
    if (threadIdx.x == 0) s_missing = 0;
    __syncthreads();
    if (threadIdx.x < world) {
        const volatile int *flag = flags + half * world + threadIdx.x;
        int polls = 0;
        while (*flag < call && polls < wait_limit) {
            __nanosleep(256);
            polls++;
        }
        if (*flag < call) atomicAdd(&s_missing, 1);
    }
    __syncthreads();
    if (s_missing != 0) {   // some rank never arrived: report it, leave the values alone
        if (threadIdx.x == 0) atomicOr(status, MCTSNC_EXCHANGE_TIMEOUT);
        return;
    }
    __threadfence_system();
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        long long acc = 0;
        for (int r = 0; r < world; r++) acc += __ldcv(data + ((long long)half * world + r) * n_max + i);
        values[i] = acc;
    }
}

}  // namespace

struct mctsnc_exchange {
    int rank = 0, world = 1, device = 0, call = 0;
    long long n_max = 0;
    char *local = nullptr;      // one allocation: data, then flags, then the status word
    size_t data_bytes = 0, flag_bytes = 0;
    void *opened[MAX_WORLD] = {};
    PeerTable peers = {};
    bool connected = false;
};

static long long *data_of(char *base) { return reinterpret_cast<long long *>(base); }
static int *flags_of(const mctsnc_exchange *ex, char *base) { return reinterpret_cast<int *>(base + ex->data_bytes); }
static int *status_of(const mctsnc_exchange *ex) { return reinterpret_cast<int *>(ex->local + ex->data_bytes + ex->flag_bytes); }

extern "C" int mctsnc_exchange_create(int32_t rank, int32_t world, int64_t n_values_max, int32_t device, mctsnc_exchange **out,
                                      unsigned char *ipc_handle_out) {
    if (!out || !ipc_handle_out || world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || n_values_max < 1)
        return MCTSNC_E_BAD_ARGUMENT;
    *out = nullptr;
    CUDA_TRY(cudaSetDevice(device));
    mctsnc_exchange *ex = new (std::nothrow) mctsnc_exchange();
    if (!ex) return MCTSNC_E_NO_MEMORY;
    ex->rank = rank;
    ex->world = world;
    ex->device = device;
    ex->n_max = n_values_max;
    ex->data_bytes = sizeof(long long) * 2 * (size_t)world * (size_t)n_values_max;
    ex->flag_bytes = sizeof(int) * 2 * (size_t)world;
    const size_t total = ex->data_bytes + ex->flag_bytes + 16;
    cudaError_t e = cudaMalloc((void **)&ex->local, total);
    if (e == cudaSuccess) e = cudaMemset(ex->local, 0, total);
    cudaIpcMemHandle_t handle;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&handle, ex->local);
    if (e != cudaSuccess) {
        cudaFree(ex->local);
        delete ex;
        cudaGetLastError();
        return (int)e;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == MCTSNC_EXCHANGE_HANDLE_BYTES, "handle size quoted in the header");
    for (size_t i = 0; i < sizeof(handle); i++) ipc_handle_out[i] = reinterpret_cast<unsigned char *>(&handle)[i];
    *out = ex;
    return 0;
}

extern "C" int mctsnc_exchange_connect(mctsnc_exchange *ex, const unsigned char *all_handles) {
    if (!ex || ex->connected) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(ex->device));
    for (int r = 0; r < ex->world; r++) {
        char *base = ex->local;   // own rank, and every rank in loop-back mode (all_handles == NULL)
        if (all_handles && r != ex->rank) {
            cudaIpcMemHandle_t handle;
            for (size_t i = 0; i < sizeof(handle); i++)
                reinterpret_cast<unsigned char *>(&handle)[i] = all_handles[(size_t)r * MCTSNC_EXCHANGE_HANDLE_BYTES + i];
            void *p = nullptr;
            CUDA_TRY(cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess));
            ex->opened[r] = p;
            base = static_cast<char *>(p);
        }
        ex->peers.data[r] = data_of(base);
        ex->peers.flags[r] = flags_of(ex, base);
    }
    ex->connected = true;
    return 0;
}

extern "C" int mctsnc_exchange_allreduce(mctsnc_exchange *ex, int64_t *values_device, int64_t n, int32_t wait_limit, void *stream) {
    if (!ex || !ex->connected || !values_device || n < 1 || wait_limit < 1) return MCTSNC_E_BAD_ARGUMENT;
    if (n > ex->n_max) return MCTSNC_E_CAPACITY;
    CUDA_TRY(cudaSetDevice(ex->device));
    cudaStream_t s = (cudaStream_t)stream;
    ex->call += 1;
    push_kernel<<<1, EXCHANGE_THREADS, 0, s>>>(ex->peers, (const long long *)values_device, n, ex->n_max, ex->rank, ex->world, ex->call);
    sum_kernel<<<1, EXCHANGE_THREADS, 0, s>>>(data_of(ex->local), flags_of(ex, ex->local), (long long *)values_device, n, ex->n_max,
                                              ex->world, ex->call, wait_limit, status_of(ex));
    return (int)cudaGetLastError();
}

extern "C" int mctsnc_exchange_status(mctsnc_exchange *ex, int32_t *status_out, void *stream) {
    if (!ex || !status_out) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(ex->device));
    cudaStream_t s = (cudaStream_t)stream;
    int status = 0;
    CUDA_TRY(cudaMemcpyAsync(&status, status_of(ex), sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    *status_out = status;
    return 0;
}

extern "C" int mctsnc_exchange_destroy(mctsnc_exchange *ex) {
    if (!ex) return MCTSNC_E_BAD_ARGUMENT;
    cudaSetDevice(ex->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < ex->world; r++)
        if (ex->opened[r]) cudaIpcCloseMemHandle(ex->opened[r]);
    cudaFree(ex->local);
    delete ex;
    return 0;
}
