// Host side of libmctsnc_b200.so: the C ABI declared in include/mctsnc_b200.h, the handle that owns the device
// memory of a searcher, the random-stream set-up, the two reduction kernels and the export of trees in the
// reference's array formats.
#include "../../include/mctsnc_b200.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <mutex>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "c4_search.cuh"
#include "common.cuh"
#include "gomoku_search.cuh"
#include "rng.cuh"

using namespace mctsnc;

namespace {

constexpr int MAX_TREE_DEPTH = 2048;  // src/mctsnc.py:197
#ifndef MCTSNC_C4_CLUSTER_MIN_GAMES
#define MCTSNC_C4_CLUSTER_MIN_GAMES 256    // Connect 4: clusters only for steps with more games than this
#endif
#ifndef MCTSNC_C4_CACHE_NODES
#define MCTSNC_C4_CACHE_NODES 6144      // Connect-4 cluster kernel, one block per SM: node records kept in shared memory
#endif
#ifndef MCTSNC_C4_CLUSTER_SM_SHARE
#define MCTSNC_C4_CLUSTER_SM_SHARE 4   // Connect 4: clusters of blocks per tree while they make at most this many blocks per SM
#endif
constexpr int GOMOKU_STREAMS = 8;     // tree groups of a Gomoku search launch that run out of step with each other

#define CUDA_TRY(expr)                        \
    do {                                      \
        cudaError_t _e = (expr);              \
        if (_e != cudaSuccess) return (int)_e; \
    } while (0)

int pow2ceil(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

// device-side result block of one search, filled by the two reduction kernels
struct DevResult {
    int best_action;
    int best_win_flag;
    long long best_n;
    long long best_n_wins;
    long long playouts;
    long long plies;
    long long ub_draws;
    unsigned status;
    int n_root_actions;
    int max_depth;
    int max_size;
    long long total_nodes;
    long long depth_sum;
    float stage_ms[4];   // mean over the search's trees of TreeState::stage_ms
};

}  // namespace

struct mctsnc_handle {
    mctsnc_config cfg;
    int A = 0;
    int tpb_e1 = 0;
    int tpb_roa = 0;
    int sm_count = 0;
    bool cluster_ok = false;      // thread-block clusters can be launched (and MCTSNC_B200_NO_CLUSTER is not set)
    int cluster_fit[2] = {0, 0};  // clusters that fit on the device at once, by record-cache size (0: not asked yet, -1: unknown)
    int threads = 0;
    int blocks_per_sm = 0;
    long long bytes = 0;
    long long n_trees_total = 0;  // max_batch * n_trees
    long long rng_per_search = 0; // playout streams per search of this handle
    // device memory
    int4 *rec = nullptr;
    ulonglong2 *board = nullptr;
    int *parent = nullptr;
    TreeState *state = nullptr;
    int *paths = nullptr;
    short *actions_expanded = nullptr;
    int *child_out = nullptr;
    ulonglong2 *rng_playout = nullptr;
    ulonglong2 *rng_expand = nullptr;
    ulonglong2 *rng_playout_base = nullptr;
    ulonglong2 *rng_expand_base = nullptr;
    JumpColumn *jump_cols = nullptr;      // [JUMP_LEVELS][128] matrices of the 2^64-step jump, for seeding streams on the device
    ulonglong2 *root_board = nullptr;
    signed char *root_turn = nullptr;
    WorkQueues *queue = nullptr;          // Connect 4: work queue of batched launches
    QueueCell *ring = nullptr;            // [QUEUE_LEVELS][n_trees_total]
    int *remaining = nullptr;             // [n_trees_total]
    long long *trace = nullptr;           // optional slice record of queued launches: [trace_cap][4]
    int *trace_count = nullptr;
    int trace_cap = 0;
    // Gomoku only
    unsigned *gboard = nullptr;           // [trees][cap][16]
    gomoku::StepInfo *gstep = nullptr;    // [trees]
    unsigned *gtpl = nullptr;             // [trees][gomoku::TPL_WORDS]
    int *path_ns = nullptr, *path_wins = nullptr;
    signed char *child_outcome = nullptr;
    unsigned char *child_action = nullptr;
    unsigned char *active_rank = nullptr;
    unsigned *root_gboard = nullptr;      // [max_batch][16]
    unsigned *h_root_gboard = nullptr;
    long long *sums = nullptr;            // [max_batch][3A]
    unsigned char *flags = nullptr;       // [max_batch][2A]: win flags, expanded-at-root
    DevResult *dres = nullptr;            // [max_batch]
    // pinned host staging
    ulonglong2 *h_root_board = nullptr;
    signed char *h_root_turn = nullptr;
    long long *h_sums = nullptr;
    unsigned char *h_flags = nullptr;
    DevResult *h_dres = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaEvent_t ev_staged = nullptr;  // recorded behind the host-to-device copies of the staged roots
    bool staging_in_flight = false;
    float last_ms = 0.f;
    long long last_steps = 0;
    // Gomoku: streams of the tree groups of a search launch, with the events that fork them from and join them to the
    // caller's stream
    cudaStream_t g_stream[GOMOKU_STREAMS] = {};
    cudaEvent_t g_fork = nullptr, g_join[GOMOKU_STREAMS] = {};
    float ms_per_cycle = 0.f;  // 1 / nominal SM clock in kHz
    cudaEvent_t ev_r0 = nullptr, ev_r1 = nullptr;  // behind the two reduction kernels of mctsnc_run
    float reduce_ms[2] = {0.f, 0.f};
    int staged_roots = 0;  // roots resident on the device from the last staging
    size_t dyn_smem = 0;   // dynamic shared memory of the search kernel: the tree's random streams
};

namespace {

// ---------------------------------------------------------------------------------------------------------------
// kernels outside the search loop

// fills the work queue of a batched launch with every tree once (in the highest ring: nothing is known yet about the
// work a tree has), each with `steps` steps to do
__global__ void init_queue_kernel(WorkQueues *q, QueueCell *rings, int *remaining, int trees, int steps) {
    const int gsz = gridDim.x * blockDim.x;
    const int gid = blockIdx.x * blockDim.x + threadIdx.x;
    for (int i = gid; i < trees * QUEUE_LEVELS; i += gsz) {
        const int level = i / trees, c = i - level * trees;
        const bool top = level == QUEUE_LEVELS - 1;
        rings[i].tree = top ? c : -1;
        rings[i].seq = top ? c + 1 : c;
    }
    for (int i = gid; i < trees; i += gsz) remaining[i] = steps;
    if (gid < QUEUE_LEVELS) {  // blocks have 256 threads
        q->level[gid].head = 0;
        q->level[gid].tail = gid == QUEUE_LEVELS - 1 ? trees : 0;
    }
    if (gid == 0) {
        q->nonempty = 1ULL << (QUEUE_LEVELS - 1);
        q->longest_us = 0;
    }
}

// after a queued launch: a tree that still has steps to do was lost by the queue; report it instead of returning a
// short search
__global__ void check_queue_kernel(const int *remaining, TreeState *state, int trees) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < trees; i += gridDim.x * blockDim.x)
        if (remaining[i] != 0) atomicOr(&state[i].status, STATUS_INTERNAL);
}

// copies the freshly seeded streams of one search into the slots of `batch` searches
__global__ void replicate_streams_kernel(ulonglong2 *dst, const ulonglong2 *base, long long per_search, int batch) {
    const long long n = per_search * batch;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = base[i % per_search];
}

// _reduce_over_trees_* (src/mctsnc.py:2223-2296): per root action the sums over the trees of a search of the root
// visit count, the child's visit count and the child's win count; win flag from tree 0.  One block per search.
// Also gathers the statistics behind performance_info (:448-494).
__global__ void reduce_over_trees_kernel(const int4 *rec, const TreeState *state, long long cap, int n_trees, int A,
                                         long long *sums, unsigned char *flags, DevResult *dres) {
    const int b = blockIdx.x;
    const int tid = threadIdx.x;
    const int4 *r0 = rec + (long long)b * n_trees * cap;
    const int root_meta0 = r0[0].w;
    const int root_turn = meta_turn(root_meta0);
    const unsigned mask0 = root_meta0 & 0x7F;
    for (int a = tid; a < A; a += blockDim.x) {
        long long s_root = 0, s_n = 0, s_w = 0;
        unsigned char win = 0;
        const bool expanded = (mask0 >> a) & 1u;
        if (expanded) {
            for (int t = 0; t < n_trees; t++) {
                const int4 *rt = r0 + (long long)t * cap;
                const int4 root = rt[0];
                s_root += root.x;
                const unsigned mk = root.w & 0x7F;
                if ((mk >> a) & 1u) {
                    const int4 c = rt[root.z + __popc(mk & ((1u << a) - 1u))];
                    s_n += c.x;
                    s_w += c.y;
                    if (t == 0) win = (c.w & META_TERMINAL) && meta_outcome(c.w) == root_turn;
                }
            }
        }
        sums[(long long)b * 3 * A + a] = s_root;
        sums[(long long)b * 3 * A + A + a] = s_n;
        sums[(long long)b * 3 * A + 2 * A + a] = s_w;
        flags[(long long)b * 2 * A + a] = win;
        flags[(long long)b * 2 * A + A + a] = expanded;
    }
    // statistics
    __shared__ long long sh_depth[256];
    __shared__ int sh_maxd[256];
    long long dsum = 0;
    int dmax = 0;
    for (int t = 0; t < n_trees; t++) {
        const int size = state[b * n_trees + t].size;
        const int4 *rt = r0 + (long long)t * cap;
        for (int i = tid; i < size; i += blockDim.x) {
            const int d = meta_depth(rt[i].w);
            dsum += d;
            dmax = d > dmax ? d : dmax;
        }
    }
    sh_depth[tid] = dsum;
    sh_maxd[tid] = dmax;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (tid < s) {
            sh_depth[tid] += sh_depth[tid + s];
            sh_maxd[tid] = max(sh_maxd[tid], sh_maxd[tid + s]);
        }
        __syncthreads();
    }
    if (tid == 0) {
        DevResult d;
        d.best_action = -1;
        d.best_win_flag = 0;
        d.best_n = 0;
        d.best_n_wins = 0;
        d.playouts = 0;
        d.plies = 0;
        d.ub_draws = 0;
        d.status = 0;
        d.max_size = 0;
        d.total_nodes = 0;
        for (int t = 0; t < n_trees; t++) {
            const TreeState &ts = state[b * n_trees + t];
            d.playouts += r0[(long long)t * cap].x;
            d.plies += (long long)ts.plies;
            d.ub_draws += (long long)ts.ub_draws;
            d.status |= ts.status;
            d.total_nodes += ts.size;
            d.max_size = ts.size > d.max_size ? ts.size : d.max_size;
        }
        d.n_root_actions = __popc(mask0);
        d.max_depth = sh_maxd[0];
        d.depth_sum = sh_depth[0];
        for (int k = 0; k < 4; k++) {
            float acc = 0.f;
            for (int t = 0; t < n_trees; t++) acc += state[b * n_trees + t].stage_ms[k];
            d.stage_ms[k] = acc / (float)n_trees;
        }
        dres[b] = d;
    }
}

// _reduce_over_actions_* (src/mctsnc.py:2299-2375): lexicographic max/argmax over (win_flag, n, n_wins) with the
// reference's stride-halving reduction, which keeps the left operand on ties.  The thrifty variants reduce over
// ordinals among the root's expanded actions, the prodigal ones over action indices.  One block of `width` threads
// per search (width = tpb_roa).
__global__ void reduce_over_actions_kernel(const long long *sums, const unsigned char *flags, int A, int width, int thrifty,
                                           DevResult *dres) {
    __shared__ short s_a[512];
    __shared__ unsigned char s_f[512];
    __shared__ long long s_n[512];
    __shared__ long long s_w[512];
    __shared__ short s_ord2act[512];
    __shared__ int s_cnt;
    const int b = blockIdx.x;
    const int t = threadIdx.x;
    const long long *sm = sums + (long long)b * 3 * A;
    const unsigned char *fl = flags + (long long)b * 2 * A;
    if (t == 0) {
        int c = 0;
        for (int a = 0; a < A; a++)
            if (fl[A + a]) s_ord2act[c++] = (short)a;
        s_cnt = c;
    }
    __syncthreads();
    const int limit = thrifty ? s_cnt : A;
    const int src = thrifty ? (t < limit ? s_ord2act[t] : 0) : t;
    s_a[t] = (short)t;
    if (t < limit) {
        s_f[t] = fl[src];
        s_n[t] = sm[A + src];
        s_w[t] = sm[2 * A + src];
    } else {
        s_f[t] = 0;
        s_n[t] = 0;
        s_w[t] = 0;
    }
    __syncthreads();
    for (int stride = width >> 1; stride > 0; stride >>= 1) {
        if (t < stride) {
            const int o = t + stride;
            if ((s_f[t] < s_f[o]) || (s_f[t] == s_f[o] && s_n[t] < s_n[o]) ||
                (s_f[t] == s_f[o] && s_n[t] == s_n[o] && s_w[t] < s_w[o])) {
                s_a[t] = s_a[o];
                s_f[t] = s_f[o];
                s_n[t] = s_n[o];
                s_w[t] = s_w[o];
            }
        }
        __syncthreads();
    }
    if (t == 0) {
        int best = s_a[0];
        if (thrifty) best = best < s_cnt ? s_ord2act[best] : 0;
        dres[b].best_action = best;
        dres[b].best_win_flag = s_f[0];
        dres[b].best_n = s_n[0];
        dres[b].best_n_wins = s_w[0];
    }
}

// _reduce_over_trees_* for Gomoku nodes (first child + number of children; the child of action a is found through the
// empty cells of the root position)
__global__ void gomoku_reduce_over_trees_kernel(const int4 *rec, const unsigned *board, const TreeState *state, long long cap,
                                                int n_trees, long long *sums, unsigned char *flags, DevResult *dres) {
    constexpr int A = gomoku::A;
    const int b = blockIdx.x;
    const int tid = threadIdx.x;
    const int4 *r0 = rec + (long long)b * n_trees * cap;
    const unsigned *b0 = board + (long long)b * n_trees * cap * 16;   // root position (the same in every tree)
    __shared__ unsigned s_empty[8];
    __shared__ int s_prefix[9];
    if (tid < 8) s_empty[tid] = ~(b0[tid] | b0[8 + tid]) & (tid == 7 ? 0x1u : 0xFFFFFFFFu);
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int w = 0; w < 8; w++) {
            s_prefix[w] = acc;
            acc += __popc(s_empty[w]);
        }
        s_prefix[8] = acc;
    }
    __syncthreads();
    const int root_turn = gomoku::g_turn(r0[0].w);
    const int n_children0 = r0[0].w & gomoku::G_NCHILD_MASK;
    for (int a = tid; a < A; a += blockDim.x) {
        long long s_root = 0, s_n = 0, s_w = 0;
        unsigned char win = 0;
        const int w = a >> 5, bit = a & 31;
        const int rank = s_prefix[w] + __popc(s_empty[w] & ((1u << bit) - 1u));
        const bool expanded = ((s_empty[w] >> bit) & 1u) && rank < n_children0;
        if (expanded) {
            for (int t = 0; t < n_trees; t++) {
                const int4 *rt = r0 + (long long)t * cap;
                const int4 root = rt[0];
                s_root += root.x;
                if (rank < (root.w & gomoku::G_NCHILD_MASK)) {
                    const int4 c = rt[root.z + rank];
                    s_n += c.x;
                    s_w += c.y;
                    if (t == 0) win = (c.w & gomoku::G_TERMINAL) && gomoku::g_outcome(c.w) == root_turn;
                }
            }
        }
        sums[(long long)b * 3 * A + a] = s_root;
        sums[(long long)b * 3 * A + A + a] = s_n;
        sums[(long long)b * 3 * A + 2 * A + a] = s_w;
        flags[(long long)b * 2 * A + a] = win;
        flags[(long long)b * 2 * A + A + a] = expanded;
    }
    __shared__ long long sh_depth[256];
    __shared__ int sh_maxd[256];
    long long dsum = 0;
    int dmax = 0;
    for (int t = 0; t < n_trees; t++) {
        const int size = state[b * n_trees + t].size;
        const int4 *rt = r0 + (long long)t * cap;
        for (int i = tid; i < size; i += blockDim.x) {
            const int d = meta_depth(rt[i].w);
            dsum += d;
            dmax = d > dmax ? d : dmax;
        }
    }
    sh_depth[tid] = dsum;
    sh_maxd[tid] = dmax;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (tid < s) {
            sh_depth[tid] += sh_depth[tid + s];
            sh_maxd[tid] = max(sh_maxd[tid], sh_maxd[tid + s]);
        }
        __syncthreads();
    }
    if (tid == 0) {
        DevResult d;
        d.best_action = -1;
        d.best_win_flag = 0;
        d.best_n = 0;
        d.best_n_wins = 0;
        d.playouts = 0;
        d.plies = 0;
        d.ub_draws = 0;
        d.status = 0;
        d.max_size = 0;
        d.total_nodes = 0;
        for (int t = 0; t < n_trees; t++) {
            const TreeState &ts = state[b * n_trees + t];
            d.playouts += r0[(long long)t * cap].x;
            d.plies += (long long)ts.plies;
            d.ub_draws += (long long)ts.ub_draws;
            d.status |= ts.status;
            d.total_nodes += ts.size;
            d.max_size = ts.size > d.max_size ? ts.size : d.max_size;
        }
        d.n_root_actions = n_children0;
        d.max_depth = sh_maxd[0];
        d.depth_sum = sh_depth[0];
        for (int k = 0; k < 4; k++) {
            float acc = 0.f;
            for (int t = 0; t < n_trees; t++) acc += state[b * n_trees + t].stage_ms[k];
            d.stage_ms[k] = acc / (float)n_trees;
        }
        dres[b] = d;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host helpers

// create_xoroshiro128p_states(n, seed) restricted to the streams [first, first + count) with stride `stride`
// between wanted streams (stream i is stream i-1 jumped 2^64 steps ahead)
void make_streams(uint64_t seed, long long first, long long count, long long stride, ulonglong2 *out) {
    RngState s;
    rng_seed(s, seed);
    long long idx = 0;
    for (long long k = 0; k < count; k++) {
        const long long want = first + k * stride;
        while (idx < want) {
            rng_jump(s);
            idx++;
        }
        out[k].x = s.s0;
        out[k].y = s.s1;
    }
}

// the jump matrices, computed once per process
const JumpColumn *jump_matrix_table() {
    static JumpColumn table[JUMP_LEVELS * 128];
    static std::once_flag once;
    std::call_once(once, [] { jump_matrices(table); });
    return table;
}

bool is_ocp(const mctsnc_config &c) { return c.variant == MCTSNC_OCP_THRIFTY || c.variant == MCTSNC_OCP_PRODIGAL; }
bool is_thrifty(const mctsnc_config &c) { return c.variant == MCTSNC_OCP_THRIFTY || c.variant == MCTSNC_ACP_THRIFTY; }

// int8 board + column fills -> bitboards; rejects positions the bitboard mechanics cannot represent
int c4_encode_root(const int8_t *board, const int8_t *fills, ulonglong2 *out) {
    unsigned long long neg = 0, pos = 0;
    for (int j = 0; j < c4::COLS; j++) {
        int f = 0;
        bool gap = false;
        for (int h = 0; h < c4::ROWS; h++) {
            const int v = board[(c4::ROWS - 1 - h) * c4::COLS + j];
            if (v == 0) {
                gap = true;
                continue;
            }
            if (gap || (v != 1 && v != -1)) return MCTSNC_E_BAD_ROOT;  // a disc above an empty cell
            if (v > 0) pos |= 1ULL << (7 * j + h);
            else neg |= 1ULL << (7 * j + h);
            f++;
        }
        if (fills && fills[j] != f) return MCTSNC_E_BAD_ROOT;
    }
    if (c4::has_four(neg) || c4::has_four(pos)) return MCTSNC_E_BAD_ROOT;  // the game is over already
    out->x = neg;
    out->y = pos;
    return 0;
}

// int8 board -> two 225-bit stone sets (cell (i, j) = bit i*15+j)
int gomoku_encode_root(const int8_t *board, unsigned *out) {
    for (int k = 0; k < 16; k++) out[k] = 0;
    for (int c = 0; c < gomoku::A; c++) {
        const int v = board[c];
        if (v == -1) out[c >> 5] |= 1u << (c & 31);
        else if (v == 1) out[8 + (c >> 5)] |= 1u << (c & 31);
        else if (v != 0) return MCTSNC_E_BAD_ROOT;
    }
    return 0;
}

bool is_gomoku(const mctsnc_config &c) { return c.game == MCTSNC_GAME_GOMOKU; }

template <typename T>
int dev_alloc(mctsnc_handle *h, T **p, long long n) {
    if (n <= 0) n = 1;
    cudaError_t e = cudaMalloc((void **)p, (size_t)n * sizeof(T));
    if (e != cudaSuccess) {
        *p = nullptr;
        cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? MCTSNC_E_NO_MEMORY : (int)e;
    }
    h->bytes += n * (long long)sizeof(T);
    return 0;
}

void release(mctsnc_handle *h) {
    cudaFree(h->rec);
    cudaFree(h->board);
    cudaFree(h->parent);
    cudaFree(h->state);
    cudaFree(h->paths);
    cudaFree(h->actions_expanded);
    cudaFree(h->child_out);
    cudaFree(h->rng_playout);
    cudaFree(h->rng_expand);
    cudaFree(h->rng_playout_base);
    cudaFree(h->rng_expand_base);
    cudaFree(h->jump_cols);
    cudaFree(h->root_board);
    cudaFree(h->root_turn);
    cudaFree(h->queue);
    cudaFree(h->ring);
    cudaFree(h->remaining);
    cudaFree(h->trace);
    cudaFree(h->trace_count);
    cudaFree(h->gboard);
    cudaFree(h->gstep);
    cudaFree(h->gtpl);
    cudaFree(h->path_ns);
    cudaFree(h->path_wins);
    cudaFree(h->child_outcome);
    cudaFree(h->child_action);
    cudaFree(h->active_rank);
    cudaFree(h->root_gboard);
    cudaFreeHost(h->h_root_gboard);
    cudaFree(h->sums);
    cudaFree(h->flags);
    cudaFree(h->dres);
    cudaFreeHost(h->h_root_board);
    cudaFreeHost(h->h_root_turn);
    cudaFreeHost(h->h_sums);
    cudaFreeHost(h->h_flags);
    cudaFreeHost(h->h_dres);
    if (h->ev0) cudaEventDestroy(h->ev0);
    if (h->ev1) cudaEventDestroy(h->ev1);
    if (h->ev_staged) cudaEventDestroy(h->ev_staged);
    if (h->ev_r0) cudaEventDestroy(h->ev_r0);
    if (h->ev_r1) cudaEventDestroy(h->ev_r1);
    if (h->g_fork) cudaEventDestroy(h->g_fork);
    for (int g = 0; g < GOMOKU_STREAMS; g++) {
        if (h->g_join[g]) cudaEventDestroy(h->g_join[g]);
        if (h->g_stream[g]) cudaStreamDestroy(h->g_stream[g]);
    }
}

#ifndef MCTSNC_SLICE_STEPS
#define MCTSNC_SLICE_STEPS 32
#endif
constexpr int SLICE_STEPS = MCTSNC_SLICE_STEPS;  // steps a block runs of one tree before it takes the next tree from the queue

const void *search_kernel_ptr(const mctsnc_config &c) {
    return is_ocp(c) ? (const void *)c4::search_kernel<true> : (const void *)c4::search_kernel<false>;
}

// Threads of the block that grows one tree, from the games a step plays (n_playouts, times the children of a node for
// the ACP variants) and from how many trees there are for the device.
//   Many trees (at least two per SM): a quarter of the games, between 32 and 320; half of them when a step has at most 256
//   games.  Measured on 256 roots: headline ACP
//   4 x 256 (1792 games a step) 16.9 / 18.2 / 17.3 / 15.8 / 15.7 G playouts/s at 256 / 320 / 384 / 448 / 512 threads (three
//   blocks per SM up to 384; a thread of a smaller block plays more games per step, so less of a step is spent waiting for
//   its last games); OCP 8 trees x 1000 steps with 32 / 128 / 512 playouts: 4.2 / 8.2 / 17.7 G/s at 32 / 64 / 128 threads
//   against 1.4 / 5.0 / 12.8 at 384 (small blocks put more trees on an SM, which hides the latency of the
//   select/expand/backup warp); with 8 x 1000 steps and 64 / 128 / 256 / 512 playouts, threads = playouts / 4, / 2, / 1:
//   - / 6.3 / 5.9, 8.3 / 8.6 / 7.7, 11.3 / 13.0 / 10.5, 18.6 / 15.7 / 10.7 G/s.
//   Few trees (a tree has an SM to itself): one thread per game, at most 1024; measured on one 4-tree ACP search of
//   2000 steps: 94.7 ms with 256 threads, 69.3 ms with 512, 67.5 ms with 1024.  In between: half the games, at most 512.
int choose_threads(mctsnc_handle *h, long long trees) {
    const int games = h->cfg.n_playouts * (is_ocp(h->cfg) ? 1 : h->A);
    auto fit = [](int want, int most) {
        const int t = (want + 31) / 32 * 32;
        return t < 32 ? 32 : (t > most ? most : t);
    };
    int threads;
    if (trees >= 2LL * h->sm_count) threads = fit(games <= 256 ? games / 2 : games / 4, 320);
    else if (trees <= h->sm_count) threads = fit(games, 1024);
    else threads = fit(games / 2, 512);
    const void *fn = search_kernel_ptr(h->cfg);
    int per_sm = 0;
    while (threads > 32 &&
           (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, h->dyn_smem) != cudaSuccess || per_sm < 1))
        threads -= 32;
    return threads;
}

int seed_streams(mctsnc_handle *h, int batch, cudaStream_t stream) {
    const int grid = 148 * 4;
    replicate_streams_kernel<<<grid, 256, 0, stream>>>(h->rng_playout, h->rng_playout_base, h->rng_per_search, batch);
    if (is_ocp(h->cfg))
        replicate_streams_kernel<<<grid, 256, 0, stream>>>(h->rng_expand, h->rng_expand_base, h->cfg.n_trees, batch);
    return (int)cudaGetLastError();
}

int stage_roots(mctsnc_handle *h, int batch, const int8_t *boards, const int8_t *extras, const int8_t *turns,
                cudaStream_t stream) {
    const int cells = h->cfg.board_rows * h->cfg.board_cols;
    const int extra = h->cfg.extra_info_memory;
    // the pinned staging buffers are about to be rewritten: the copies of the previous call (asynchronous entry points
    // return before they ran) must have read them
    if (h->staging_in_flight) {
        CUDA_TRY(cudaEventSynchronize(h->ev_staged));
        h->staging_in_flight = false;
    }
    if (is_gomoku(h->cfg)) {
        for (int b = 0; b < batch; b++) {
            if (turns[b] != 1 && turns[b] != -1) return MCTSNC_E_BAD_ARGUMENT;
            const int rc = gomoku_encode_root(boards + (long long)b * cells, h->h_root_gboard + (long long)b * 16);
            if (rc) return rc;
            h->h_root_turn[b] = turns[b];
        }
        CUDA_TRY(cudaMemcpyAsync(h->root_gboard, h->h_root_gboard, sizeof(unsigned) * 16 * batch, cudaMemcpyHostToDevice, stream));
        CUDA_TRY(cudaMemcpyAsync(h->root_turn, h->h_root_turn, batch, cudaMemcpyHostToDevice, stream));
        CUDA_TRY(cudaEventRecord(h->ev_staged, stream));
        h->staging_in_flight = true;
        return 0;
    }
    for (int b = 0; b < batch; b++) {
        if (turns[b] != 1 && turns[b] != -1) return MCTSNC_E_BAD_ARGUMENT;
        const int rc = c4_encode_root(boards + (long long)b * cells, extras ? extras + (long long)b * extra : nullptr,
                                      &h->h_root_board[b]);
        if (rc) return rc;
        h->h_root_turn[b] = turns[b];
    }
    CUDA_TRY(cudaMemcpyAsync(h->root_board, h->h_root_board, sizeof(ulonglong2) * batch, cudaMemcpyHostToDevice, stream));
    CUDA_TRY(cudaMemcpyAsync(h->root_turn, h->h_root_turn, batch, cudaMemcpyHostToDevice, stream));
    CUDA_TRY(cudaEventRecord(h->ev_staged, stream));
    h->staging_in_flight = true;
    return 0;
}

// Gomoku: two launches per step (tree step, playouts) and a closing backup, all enqueued without waiting.
//
// The trees are split into groups, each with a stream of its own: a tree's next step only needs that tree's games to be
// over, so the groups run out of step with each other and the lanes one tree leaves idle while its longest games finish
// (up to ~170 plies against a mean of ~85) play the games of the others.  Every playout launch asks for enough blocks
// for all its games at once; blocks whose warps find no game left return at once and make room for the blocks of the
// other groups' launches, so the device is shared by whatever games exist at the moment.  No kernel waits for another:
// the order inside a group is stream order, the groups are forked from and joined to the caller's stream with events.
int launch_search_gomoku(mctsnc_handle *h, int batch, int steps, int first, cudaStream_t stream) {
    gomoku::Params p;
    p.rec = h->rec;
    p.board = h->gboard;
    p.parent = h->parent;
    p.state = h->state;
    p.step = h->gstep;
    p.paths = h->paths;
    p.path_ns = h->path_ns;
    p.path_wins = h->path_wins;
    p.actions_expanded = h->actions_expanded;
    p.child_out = h->child_out;
    p.child_outcome = h->child_outcome;
    p.child_action = h->child_action;
    p.active_rank = h->active_rank;
    p.tpl = h->gtpl;
    p.rng_playout = h->rng_playout;
    p.rng_expand = h->rng_expand;
    p.root_board = h->root_gboard;
    p.root_turn = h->root_turn;
    p.cap = h->cfg.node_capacity;
    p.node_limit = h->cfg.max_tree_size < h->cfg.node_capacity ? h->cfg.max_tree_size : h->cfg.node_capacity;
    p.n_trees = h->cfg.n_trees;
    p.n_playouts = h->cfg.n_playouts;
    p.variant = h->cfg.variant;
    p.ucb_c = h->cfg.ucb_c;
    p.ms_per_cycle = h->ms_per_cycle;
    const int trees = (int)((long long)batch * h->cfg.n_trees);
    const bool ocp = is_ocp(h->cfg);
    // resident playout blocks: three per SM (limited by shared memory)
    int per_sm = 0;
    const void *pk = ocp ? (const void *)gomoku::playout_dynamic_kernel<true> : (const void *)gomoku::playout_dynamic_kernel<false>;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pk, gomoku::DYN_THREADS, h->dyn_smem) != cudaSuccess || per_sm < 1) per_sm = 1;
    const long long resident = (long long)per_sm * h->sm_count;
    h->threads = gomoku::DYN_THREADS;
    h->blocks_per_sm = per_sm;
    const int groups = trees < GOMOKU_STREAMS ? trees : GOMOKU_STREAMS;
    CUDA_TRY(cudaEventRecord(h->g_fork, stream));
    for (int g = 0; g < groups; g++) CUDA_TRY(cudaStreamWaitEvent(h->g_stream[g], h->g_fork, 0));
    for (int s = 0; s <= steps; s++) {
        p.first = (first && s == 0) ? 1 : 0;
        p.backup_only = s == steps ? 1 : 0;
        for (int g = 0; g < groups; g++) {
            const int t0 = (int)((long long)trees * g / groups), t1 = (int)((long long)trees * (g + 1) / groups);
            const int n = t1 - t0;
            p.tree_base = t0;
            cudaStream_t gs = h->g_stream[g];
            if (ocp) gomoku::tree_step_kernel<true><<<n, 256, 0, gs>>>(p);
            else gomoku::tree_step_kernel<false><<<n, 256, 0, gs>>>(p);
            if (s == steps) continue;
            // Blocks of the launch.  A lane for every game while that does not oversubscribe the device much (OCP: one child
            // per tree); otherwise 1.5 to 2 times the group's share of the blocks that fit on the device at once, so that a
            // lane plays several games one after the other and its warp stays full, and blocks are waiting to start
            // where another group's launch is running out of games (a step is as long as its longest chain of games, mean
            // ~85 plies, longest ~170).  Measured, 4 x 256 acp_prodigal, 500 steps, one search (4 groups) / eight searches
            // (8 groups): 1.0 times the share 90.9 / 597 ms, 1.25: 86.4 / 541, 1.5: 85.3 / 525, 2: 87.7 / 515.
            const long long games = (long long)n * h->cfg.n_playouts * (ocp ? 1 : h->A);
            const long long enough = (games + gomoku::DYN_THREADS - 1) / gomoku::DYN_THREADS;
            long long blocks = enough;
            const long long quarters = groups >= GOMOKU_STREAMS ? 8 : 6;
            if (enough * groups > (5 * resident) / 2) blocks = (quarters * resident + 4 * groups - 1) / (4 * groups);
            if (blocks > enough) blocks = enough;
            if (blocks > resident) blocks = resident;
            if (blocks < 1) blocks = 1;
            if (ocp) gomoku::playout_dynamic_kernel<true><<<(unsigned)blocks, gomoku::DYN_THREADS, h->dyn_smem, gs>>>(p, n);
            else gomoku::playout_dynamic_kernel<false><<<(unsigned)blocks, gomoku::DYN_THREADS, h->dyn_smem, gs>>>(p, n);
        }
    }
    for (int g = 0; g < groups; g++) {
        CUDA_TRY(cudaEventRecord(h->g_join[g], h->g_stream[g]));
        CUDA_TRY(cudaStreamWaitEvent(stream, h->g_join[g], 0));
    }
    return (int)cudaGetLastError();
}

int launch_search(mctsnc_handle *h, int batch, int steps, int first, cudaStream_t stream) {
    if (is_gomoku(h->cfg)) return launch_search_gomoku(h, batch, steps, first, stream);
    SearchParams p;
    p.rec = h->rec;
    p.board = h->board;
    p.parent = h->parent;
    p.state = h->state;
    p.paths = h->paths;
    p.actions_expanded = h->actions_expanded;
    p.child_out = h->child_out;
    p.rng_playout = h->rng_playout;
    p.rng_expand = h->rng_expand;
    p.root_board = h->root_board;
    p.root_turn = h->root_turn;
    p.cap = h->cfg.node_capacity;
    p.node_limit = h->cfg.max_tree_size < h->cfg.node_capacity ? h->cfg.max_tree_size : h->cfg.node_capacity;
    p.n_trees = h->cfg.n_trees;
    p.n_playouts = h->cfg.n_playouts;
    p.log2_playouts = 0;
    while ((1 << p.log2_playouts) < h->cfg.n_playouts) p.log2_playouts++;
    p.n_actions = h->A;
    p.variant = h->cfg.variant;
    p.steps = steps;
    p.first = first;
    p.ucb_c = h->cfg.ucb_c;
    p.ms_per_cycle = h->ms_per_cycle;
    p.cache_nodes = 0;
    const long long trees = (long long)batch * h->cfg.n_trees;
    p.queue = nullptr;
    p.ring = nullptr;
    p.remaining = nullptr;
    p.ring_cap = 0;
    p.chunk = 0;
    p.trace = nullptr;
    p.trace_count = nullptr;
    p.trace_cap = 0;
    // Few trees (one search, a few searches): a cluster of blocks per tree, so that the games of a step are played on
    // several SMs at once.  Measured, 4 x 256 acp_prodigal, 2000 steps, 4 / 8 / 16 / 32 searches in one launch: 31.4 / 37.2 /
    // 40.4 / 63.2 ms with clusters against 57.3 / 57.3 / 57.3 / 57.4 ms with a block of 1024 threads per tree -- up to four
    // cluster blocks per SM pay.
    // Only where a step has more than 256 games (ACP with 64 playouts or more, OCP with 512).  One search of 2000 steps, 4
    // trees, with a block / with clusters: ACP 8 / 16 / 32 / 64 / 128 / 256 / 512 playouts 19.6 / 20.2 / 22.8 / 27.6 / 38.1 /
    // 57.2 / - ms against 20.7 / 22.0 / 23.5 / 24.2 / 25.0 / 28.3 / 36.3 ms; OCP 32 / 128 / 512 playouts 19.8 / 20.7 / 28.9
    // against 20.7 / 23.4 / 25.3 ms: with few games the two cluster barriers of a step cost more than the games take.
    if (h->cfg.threads_per_tree == 0 && h->cluster_ok && h->cfg.n_playouts >= c4::CLUSTER_BLOCKS &&
        (long long)(is_ocp(h->cfg) ? 1 : h->A) * h->cfg.n_playouts > MCTSNC_C4_CLUSTER_MIN_GAMES &&
        trees * c4::CLUSTER_BLOCKS <= (long long)MCTSNC_C4_CLUSTER_SM_SHARE * h->sm_count) {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3((unsigned)(trees * c4::CLUSTER_BLOCKS));
        lc.blockDim = dim3(c4::CLUSTER_THREADS);
        lc.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = c4::CLUSTER_BLOCKS;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        lc.attrs = &attr;
        lc.numAttrs = 1;
        if (is_ocp(h->cfg)) cudaFuncSetAttribute(c4::search_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
        else cudaFuncSetAttribute(c4::search_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
        // The first records of a tree stay in the first block's shared memory: many if every block can have an SM to itself,
        // else few.  All clusters of the launch have to be on the device at once (clusters do not spread over GPCs, so fewer
        // fit than blocks / 8): a tree whose cluster waits for another to finish would take two searches' time.
        bool fits = false;
        for (int small = trees * c4::CLUSTER_BLOCKS <= h->sm_count ? 0 : 1; small < 2 && !fits; small++) {
            p.cache_nodes = small ? 2048 : MCTSNC_C4_CACHE_NODES;
            lc.dynamicSmemBytes = h->dyn_smem / c4::CLUSTER_BLOCKS + sizeof(int4) * (size_t)p.cache_nodes;
            int &fit = h->cluster_fit[small];
            if (fit == 0) {
                int n = 0;
                const cudaError_t q = is_ocp(h->cfg) ? cudaOccupancyMaxActiveClusters(&n, c4::search_cluster_kernel<true>, &lc)
                                                     : cudaOccupancyMaxActiveClusters(&n, c4::search_cluster_kernel<false>, &lc);
                if (q != cudaSuccess) cudaGetLastError();
                fit = q == cudaSuccess && n > 0 ? n : -1;
            }
            fits = fit >= trees;
        }
        if (fits) {
            h->threads = c4::CLUSTER_THREADS * c4::CLUSTER_BLOCKS;
            h->blocks_per_sm = 1;
            const cudaError_t e = is_ocp(h->cfg) ? cudaLaunchKernelEx(&lc, c4::search_cluster_kernel<true>, p)
                                                 : cudaLaunchKernelEx(&lc, c4::search_cluster_kernel<false>, p);
            if (e == cudaSuccess) return 0;
            cudaGetLastError();      // the launch was refused (nothing ran): one block per tree from now on
            h->cluster_ok = false;
        }
        p.cache_nodes = 0;
    }
    const int threads = h->cfg.threads_per_tree > 0 ? h->cfg.threads_per_tree : choose_threads(h, trees);
    h->threads = threads;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, search_kernel_ptr(h->cfg), threads, h->dyn_smem) != cudaSuccess || per_sm < 1)
        return MCTSNC_E_BAD_ARGUMENT;
    h->blocks_per_sm = per_sm;
    // More trees than blocks fit on the device at once: a persistent grid takes slices of SLICE_STEPS steps from the
    // work queue, so that trees with long games do not keep a few SMs busy after the others have run out of work
    // (measured on 1024 trees of 2000 steps, 4 x 256 acp_prodigal: 249 ms with one block per tree, 192 ms with the queue,
    // before the later changes to the playout loop).  Otherwise block b grows tree b for the whole launch.
    const long long resident = (long long)per_sm * h->sm_count;
    unsigned grid = (unsigned)trees;
    if (trees > resident && steps > SLICE_STEPS) {
        init_queue_kernel<<<(unsigned)((trees + 255) / 256), 256, 0, stream>>>(h->queue, h->ring, h->remaining, (int)trees, steps);
        p.queue = h->queue;
        p.ring = h->ring;
        p.remaining = h->remaining;
        p.ring_cap = (int)trees;
        p.chunk = SLICE_STEPS;
        if (h->trace) {
            cudaMemsetAsync(h->trace_count, 0, sizeof(int), stream);
            p.trace = h->trace;
            p.trace_count = h->trace_count;
            p.trace_cap = h->trace_cap;
        }
        grid = (unsigned)resident;
    }
    if (is_ocp(h->cfg)) c4::search_kernel<true><<<grid, threads, h->dyn_smem, stream>>>(p);
    else c4::search_kernel<false><<<grid, threads, h->dyn_smem, stream>>>(p);
    if (p.queue) check_queue_kernel<<<(unsigned)((trees + 255) / 256), 256, 0, stream>>>(h->remaining, h->state, (int)trees);
    return (int)cudaGetLastError();
}

int launch_reduce_trees(mctsnc_handle *h, int batch, long long *sums, cudaStream_t stream) {
    if (is_gomoku(h->cfg)) {
        gomoku_reduce_over_trees_kernel<<<batch, 256, 0, stream>>>(h->rec, h->gboard, h->state, h->cfg.node_capacity,
                                                                  h->cfg.n_trees, sums, h->flags, h->dres);
        return (int)cudaGetLastError();
    }
    reduce_over_trees_kernel<<<batch, 256, 0, stream>>>(h->rec, h->state, h->cfg.node_capacity, h->cfg.n_trees, h->A, sums,
                                                        h->flags, h->dres);
    return (int)cudaGetLastError();
}

int launch_reduce_actions(mctsnc_handle *h, int batch, const long long *sums, cudaStream_t stream) {
    reduce_over_actions_kernel<<<batch, h->tpb_roa, 0, stream>>>(sums, h->flags, h->A, h->tpb_roa, is_thrifty(h->cfg) ? 1 : 0,
                                                                 h->dres);
    return (int)cudaGetLastError();
}

int fetch_results(mctsnc_handle *h, int batch, const long long *sums_dev, mctsnc_result *results, cudaStream_t stream) {
    const int A = h->A;
    CUDA_TRY(cudaMemcpyAsync(h->h_sums, sums_dev, sizeof(long long) * 3 * A * batch, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaMemcpyAsync(h->h_flags, h->flags, (size_t)2 * A * batch, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaMemcpyAsync(h->h_dres, h->dres, sizeof(DevResult) * batch, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));
    for (int b = 0; b < batch; b++) {
        mctsnc_result &r = results[b];
        const DevResult &d = h->h_dres[b];
        memset(&r, 0, sizeof(r));
        r.best_action = d.best_action;
        r.best_win_flag = d.best_win_flag;
        r.best_n = d.best_n;
        r.best_n_wins = d.best_n_wins;
        r.steps = h->last_steps;
        r.playouts = d.playouts;
        r.plies = d.plies;
        r.ub_draws = d.ub_draws;
        r.status = d.status;
        r.n_root_actions = d.n_root_actions;
        r.device_ms = h->last_ms;
        r.max_depth = d.max_depth;
        r.total_nodes = d.total_nodes;
        r.depth_sum = d.depth_sum;
        r.max_size = d.max_size;
        for (int k = 0; k < 4; k++) r.stage_ms[k] = d.stage_ms[k];
        if (is_gomoku(h->cfg)) {
            // the playouts of a Gomoku step run in a kernel of their own, shared by all trees: their time is what is left of
            // the loop after the per-tree stages
            const float rest = h->last_ms - (d.stage_ms[0] + d.stage_ms[1] + d.stage_ms[3]);
            r.stage_ms[2] = rest > 0.f ? rest : 0.f;
        }
        r.reduce_ms[0] = h->reduce_ms[0];
        r.reduce_ms[1] = h->reduce_ms[1];
        for (int a = 0; a < A; a++) {
            r.root_ns[a] = h->h_sums[(long long)b * 3 * A + a];
            r.actions_ns[a] = h->h_sums[(long long)b * 3 * A + A + a];
            r.actions_ns_wins[a] = h->h_sums[(long long)b * 3 * A + 2 * A + a];
            r.actions_win_flags[a] = h->h_flags[(long long)b * 2 * A + a];
            r.actions_expanded[a] = h->h_flags[(long long)b * 2 * A + A + a];
        }
    }
    return 0;
}

}  // namespace

// ===================================================================================================================
// C ABI

extern "C" int mctsnc_create(const mctsnc_config *cfg, mctsnc_handle **out) {
    if (!cfg || !out) return MCTSNC_E_BAD_ARGUMENT;
    *out = nullptr;
    const mctsnc_config &c = *cfg;
    if (c.variant < 0 || c.variant > 3 || c.n_trees < 1 || c.n_trees > 512 || c.n_playouts < 1 || c.n_playouts > 512 ||
        (c.n_playouts & (c.n_playouts - 1)) != 0 || c.max_batch < 1 || c.node_capacity < 2 || c.max_tree_size < 1 ||
        c.max_actions < 1 || c.max_actions > MCTSNC_MAX_ACTIONS || c.tree_offset < 0 ||
        c.n_trees_global < c.tree_offset + c.n_trees || !(c.ucb_c >= 0.f))
        return MCTSNC_E_BAD_ARGUMENT;
    if (c.threads_per_tree != 0 && (c.threads_per_tree < 32 || c.threads_per_tree > 1024 || c.threads_per_tree % 32))
        return MCTSNC_E_BAD_ARGUMENT;
    if (c.game == MCTSNC_GAME_C4) {
        if (c.board_rows != c4::ROWS || c.board_cols != c4::COLS || c.max_actions != c4::A || c.extra_info_memory != c4::COLS)
            return MCTSNC_E_UNSUPPORTED;
    } else if (c.game == MCTSNC_GAME_GOMOKU) {
        if (c.board_rows != gomoku::M || c.board_cols != gomoku::N || c.max_actions != gomoku::A || c.extra_info_memory > 1)
            return MCTSNC_E_UNSUPPORTED;
    } else {
        return MCTSNC_E_UNSUPPORTED;
    }
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev < 1) {
        cudaGetLastError();
        return MCTSNC_E_NO_DEVICE;
    }
    if (c.device < 0 || c.device >= n_dev) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(c.device));
    mctsnc_handle *h = new (std::nothrow) mctsnc_handle();
    if (!h) return MCTSNC_E_NO_MEMORY;
    h->cfg = c;
    if (h->cfg.node_capacity > h->cfg.max_tree_size) h->cfg.node_capacity = h->cfg.max_tree_size;
    if (h->cfg.node_capacity < 2) h->cfg.node_capacity = 2;
    h->A = c.max_actions;
    // tpb table of the reference, src/mctsnc.py:360-370 (only the entries that influence results)
    const int tpb_board = pow2ceil(c.board_rows * c.board_cols);
    const int tpb_extra = pow2ceil(c.extra_info_memory < 1 ? 1 : c.extra_info_memory);
    const int tpb_actions = pow2ceil(c.max_actions);
    int tpb_r = tpb_board > tpb_extra ? tpb_board : tpb_extra;
    if (tpb_r > 512) tpb_r = 512;
    h->tpb_e1 = tpb_r > tpb_actions ? tpb_r : tpb_actions;
    if (h->tpb_e1 > 512) h->tpb_e1 = 512;
    h->tpb_roa = tpb_actions;
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, c.device));
    h->sm_count = prop.multiProcessorCount;
    {
        int can = 0;
        const char *off = getenv("MCTSNC_B200_NO_CLUSTER");
        h->cluster_ok = cudaDeviceGetAttribute(&can, cudaDevAttrClusterLaunch, c.device) == cudaSuccess && can != 0 &&
                        !(off && off[0] == '1');
    }
    int clock_khz = 0;
    if (cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, c.device) != cudaSuccess || clock_khz <= 0) clock_khz = 1965000;
    h->ms_per_cycle = 1.0f / (float)clock_khz;
    h->n_trees_total = (long long)c.max_batch * c.n_trees;
    const long long nodes = h->n_trees_total * h->cfg.node_capacity;
    const bool ocp = is_ocp(c);
    h->rng_per_search = ocp ? (long long)c.n_trees * c.n_playouts : (long long)c.n_trees * h->A * c.n_playouts;
    h->dyn_smem = sizeof(ulonglong2) * (size_t)(h->rng_per_search / c.n_trees);
    if (is_gomoku(c))   // per-thread game state + per-warp templates + the tables of the exactly-five test
        h->dyn_smem = gomoku::DYN_SMEM_BYTES;
    if (h->dyn_smem > 48 * 1024) {
        const void *kernel = is_gomoku(c) ? (ocp ? (const void *)gomoku::playout_dynamic_kernel<true> : (const void *)gomoku::playout_dynamic_kernel<false>)
                                          : search_kernel_ptr(c);
        // the limit belongs to the kernel, not to the handle: never lower what another handle (or a launch) has asked for
        cudaFuncAttributes now;
        cudaError_t e = cudaFuncGetAttributes(&now, kernel);
        if (e == cudaSuccess && (size_t)now.maxDynamicSharedSizeBytes < h->dyn_smem)
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)h->dyn_smem);
        if (e != cudaSuccess) {
            delete h;
            return (int)e;
        }
    }
    int rc = 0;
    if (!rc) rc = dev_alloc(h, &h->rec, nodes);
    if (!rc && !is_gomoku(c)) rc = dev_alloc(h, &h->board, nodes);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->gboard, nodes * 16);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->gstep, h->n_trees_total);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->gtpl, h->n_trees_total * gomoku::TPL_WORDS);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->path_ns, h->n_trees_total * PATH_CAP);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->path_wins, h->n_trees_total * PATH_CAP);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->child_outcome, h->n_trees_total * h->A);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->child_action, h->n_trees_total * h->A);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->active_rank, h->n_trees_total * h->A);
    if (!rc && is_gomoku(c)) rc = dev_alloc(h, &h->root_gboard, (long long)c.max_batch * 16);
    if (!rc && is_gomoku(c) && cudaMallocHost((void **)&h->h_root_gboard, sizeof(unsigned) * 16 * c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && is_gomoku(c)) rc = (int)cudaMemset(h->gstep, 0, sizeof(gomoku::StepInfo) * h->n_trees_total);
    if (!rc && is_gomoku(c)) rc = (int)cudaMemset(h->gtpl, 0, sizeof(unsigned) * gomoku::TPL_WORDS * h->n_trees_total);
    if (!rc) rc = dev_alloc(h, &h->parent, nodes);
    if (!rc) rc = dev_alloc(h, &h->state, h->n_trees_total);
    if (!rc) rc = dev_alloc(h, &h->paths, h->n_trees_total * PATH_CAP);
    if (!rc) rc = dev_alloc(h, &h->actions_expanded, h->n_trees_total * (h->A + 2));
    if (!rc) rc = dev_alloc(h, &h->child_out, h->n_trees_total * h->A * 2);
    if (!rc) rc = dev_alloc(h, &h->rng_playout, h->rng_per_search * c.max_batch);
    if (!rc) rc = dev_alloc(h, &h->rng_playout_base, h->rng_per_search);
    if (!rc) rc = dev_alloc(h, &h->rng_expand, h->n_trees_total);
    if (!rc) rc = dev_alloc(h, &h->rng_expand_base, (long long)c.n_trees);
    if (!rc) rc = dev_alloc(h, &h->jump_cols, (long long)JUMP_LEVELS * 128);
    if (!rc) rc = (int)cudaMemcpy(h->jump_cols, jump_matrix_table(), sizeof(JumpColumn) * JUMP_LEVELS * 128, cudaMemcpyHostToDevice);
    if (!rc) rc = dev_alloc(h, &h->root_board, (long long)c.max_batch);
    if (!rc) rc = dev_alloc(h, &h->root_turn, (long long)c.max_batch);
    if (!rc && !is_gomoku(c)) rc = dev_alloc(h, &h->queue, 1);
    if (!rc && !is_gomoku(c)) rc = dev_alloc(h, &h->ring, h->n_trees_total * QUEUE_LEVELS);
    if (!rc && !is_gomoku(c)) rc = dev_alloc(h, &h->remaining, h->n_trees_total);
    if (!rc) rc = dev_alloc(h, &h->sums, (long long)c.max_batch * 3 * h->A);
    if (!rc) rc = dev_alloc(h, &h->flags, (long long)c.max_batch * 2 * h->A);
    if (!rc) rc = dev_alloc(h, &h->dres, (long long)c.max_batch);
    if (!rc && cudaMallocHost((void **)&h->h_root_board, sizeof(ulonglong2) * c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaMallocHost((void **)&h->h_root_turn, c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaMallocHost((void **)&h->h_sums, sizeof(long long) * 3 * h->A * c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaMallocHost((void **)&h->h_flags, (size_t)2 * h->A * c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaMallocHost((void **)&h->h_dres, sizeof(DevResult) * c.max_batch) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaEventCreate(&h->ev0) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaEventCreate(&h->ev1) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaEventCreateWithFlags(&h->ev_staged, cudaEventDisableTiming) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaEventCreate(&h->ev_r0) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && cudaEventCreate(&h->ev_r1) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
    if (!rc && is_gomoku(c)) {
        if (cudaEventCreateWithFlags(&h->g_fork, cudaEventDisableTiming) != cudaSuccess) rc = MCTSNC_E_NO_MEMORY;
        for (int g = 0; g < GOMOKU_STREAMS && !rc; g++)
            if (cudaStreamCreateWithFlags(&h->g_stream[g], cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&h->g_join[g], cudaEventDisableTiming) != cudaSuccess)
                rc = MCTSNC_E_NO_MEMORY;
    }
    if (!rc) rc = (int)cudaMemset(h->state, 0, sizeof(TreeState) * h->n_trees_total);
    if (!rc) rc = (int)cudaMemset(h->actions_expanded, 0, sizeof(short) * h->n_trees_total * (h->A + 2));
    if (!rc) rc = (int)cudaMemset(h->child_out, 0, sizeof(int) * h->n_trees_total * h->A * 2);
    if (rc) {
        release(h);
        delete h;
        cudaGetLastError();
        return rc;
    }
    *out = h;
    rc = mctsnc_reset_rng(h);
    if (rc) {
        mctsnc_destroy(h);
        *out = nullptr;
    }
    return rc;
}

extern "C" int mctsnc_destroy(mctsnc_handle *h) {
    if (!h) return MCTSNC_E_BAD_ARGUMENT;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    release(h);
    delete h;
    return 0;
}

extern "C" int mctsnc_reset_rng(mctsnc_handle *h) {
    if (!h) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    const mctsnc_config &c = h->cfg;
    const bool ocp = is_ocp(c);
    RngState seeded;
    rng_seed(seeded, c.seed);
    // playout streams: ACP stream (tree, action, t) = tree*A*P + action*P + t (src/mctsnc.py:1938, :2028),
    // OCP stream (tree, t) = tree*P + t (cuda.grid(1), :1849); `tree` counts over the whole (sharded) search.  Every
    // stream is computed on the device from its index (numba builds them one after the other on the host).
    const long long per_tree = ocp ? (long long)c.n_playouts : (long long)h->A * c.n_playouts;
    const unsigned grid = (unsigned)((h->rng_per_search + 127) / 128 < 4096 ? (h->rng_per_search + 127) / 128 : 4096);
    init_streams_kernel<<<grid, 128>>>(h->rng_playout_base, h->jump_cols, seeded.s0, seeded.s1, (long long)c.tree_offset * per_tree,
                                       1, h->rng_per_search);
    if (ocp)  // the child pick of tree `tree` uses stream tree * tpb_e1 of a second array with the same seed (:391, :1385)
        init_streams_kernel<<<1, 128>>>(h->rng_expand_base, h->jump_cols, seeded.s0, seeded.s1,
                                        (long long)c.tree_offset * h->tpb_e1, h->tpb_e1, c.n_trees);
    CUDA_TRY(cudaGetLastError());
    int rc = seed_streams(h, c.max_batch, 0);
    if (rc) return rc;
    CUDA_TRY(cudaDeviceSynchronize());
    return 0;
}

extern "C" int mctsnc_run(mctsnc_handle *h, const int8_t *board, const int8_t *extra_info, int32_t turn, int64_t steps_limit,
                          double time_limit_s, mctsnc_result *out) {
    if (!h || !board || !out) return MCTSNC_E_BAD_ARGUMENT;
    if (steps_limit < 0 && !(time_limit_s > 0)) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    const int8_t t8 = (int8_t)turn;
    h->staged_roots = 0;
    int rc = stage_roots(h, 1, board, extra_info, &t8, 0);
    if (rc) return rc;
    h->staged_roots = 1;
    const auto t0 = std::chrono::steady_clock::now();
    long long done = 0;
    float total_ms = 0.f;
    int chunk = steps_limit >= 0 && !(time_limit_s > 0) ? (int)(steps_limit > 1000000 ? 1000000 : steps_limit) : 16;
    int first = 1;
    for (;;) {
        bool stop = steps_limit >= 0 && done >= steps_limit;
        if (!stop && time_limit_s > 0) {
            const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            stop = el >= time_limit_s;
        }
        if (stop && !first) break;
        long long n = stop ? 0 : chunk;  // a search without a single step still resets the trees to the root
        if (steps_limit >= 0 && done + n > steps_limit) n = steps_limit - done;
        CUDA_TRY(cudaEventRecord(h->ev0, 0));
        rc = launch_search(h, 1, (int)n, first, 0);
        if (rc) return rc;
        CUDA_TRY(cudaEventRecord(h->ev1, 0));
        CUDA_TRY(cudaEventSynchronize(h->ev1));
        float ms = 0.f;
        CUDA_TRY(cudaEventElapsedTime(&ms, h->ev0, h->ev1));
        total_ms += ms;
        done += n;
        first = 0;
        if (stop) break;
        if (time_limit_s > 0 && n > 0) {
            // aim at launches of about 2 ms so that the clock is read often enough
            const double per_step = ms / (double)n;
            int next = per_step > 0 ? (int)(2.0 / per_step) : chunk * 2;
            if (next < 1) next = 1;
            if (next > 4096) next = 4096;
            chunk = next;
        }
    }
    h->last_ms = total_ms;
    h->last_steps = done;
    rc = launch_reduce_trees(h, 1, h->sums, 0);
    if (rc) return rc;
    CUDA_TRY(cudaEventRecord(h->ev_r0, 0));
    rc = launch_reduce_actions(h, 1, h->sums, 0);
    if (rc) return rc;
    CUDA_TRY(cudaEventRecord(h->ev_r1, 0));
    CUDA_TRY(cudaEventSynchronize(h->ev_r1));
    CUDA_TRY(cudaEventElapsedTime(&h->reduce_ms[0], h->ev1, h->ev_r0));
    CUDA_TRY(cudaEventElapsedTime(&h->reduce_ms[1], h->ev_r0, h->ev_r1));
    return fetch_results(h, 1, h->sums, out, 0);
}

extern "C" int mctsnc_launch_batch_device(mctsnc_handle *h, int32_t batch, const int8_t *boards, const int8_t *extras,
                                         const int8_t *turns, int64_t steps, int32_t reseed, void *stream) {
    if (!h || (boards && !turns) || batch < 1 || steps < 0 || steps > 0x7fffffff) return MCTSNC_E_BAD_ARGUMENT;
    if (batch > h->cfg.max_batch) return MCTSNC_E_CAPACITY;
    if (!boards && batch > h->staged_roots) return MCTSNC_E_BAD_ARGUMENT;  // nothing staged to search again
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    cudaStream_t s = (cudaStream_t)stream;
    int rc = 0;
    if (boards) {
        h->staged_roots = 0;
        rc = stage_roots(h, batch, boards, extras, turns, s);
        if (rc) return rc;
        h->staged_roots = batch;
    }
    if (reseed) {
        rc = seed_streams(h, batch, s);
        if (rc) return rc;
    }
    CUDA_TRY(cudaEventRecord(h->ev0, s));
    rc = launch_search(h, batch, (int)steps, 1, s);
    if (rc) return rc;
    CUDA_TRY(cudaEventRecord(h->ev1, s));
    h->last_steps = steps;
    h->reduce_ms[0] = h->reduce_ms[1] = 0.f;
    return 0;
}

extern "C" int mctsnc_reduce_trees_device(mctsnc_handle *h, int32_t batch, int64_t *partial_sums_device, void *stream) {
    if (!h || batch < 1) return MCTSNC_E_BAD_ARGUMENT;
    if (batch > h->cfg.max_batch) return MCTSNC_E_CAPACITY;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    return launch_reduce_trees(h, batch, partial_sums_device ? (long long *)partial_sums_device : h->sums, (cudaStream_t)stream);
}

extern "C" int mctsnc_search_batch_device(mctsnc_handle *h, int32_t batch, const int8_t *boards, const int8_t *extras,
                                          const int8_t *turns, int64_t steps, int32_t reseed, int64_t *partial_sums_device,
                                          void *stream) {
    int rc = mctsnc_launch_batch_device(h, batch, boards, extras, turns, steps, reseed, stream);
    if (rc) return rc;
    return mctsnc_reduce_trees_device(h, batch, partial_sums_device, stream);
}

extern "C" int mctsnc_finish_batch_device(mctsnc_handle *h, int32_t batch, const int64_t *summed_device, mctsnc_result *results,
                                          void *stream) {
    if (!h || batch < 1) return MCTSNC_E_BAD_ARGUMENT;
    if (batch > h->cfg.max_batch) return MCTSNC_E_CAPACITY;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    cudaStream_t s = (cudaStream_t)stream;
    const long long *sums = summed_device ? (const long long *)summed_device : h->sums;
    int rc = launch_reduce_actions(h, batch, sums, s);
    if (rc) return rc;
    if (!results) return 0;  // the caller keeps everything on the device
    CUDA_TRY(cudaEventSynchronize(h->ev1));
    CUDA_TRY(cudaEventElapsedTime(&h->last_ms, h->ev0, h->ev1));
    return fetch_results(h, batch, sums, results, s);
}

extern "C" int mctsnc_run_batch(mctsnc_handle *h, int32_t batch, const int8_t *boards, const int8_t *extras, const int8_t *turns,
                                int64_t steps, int32_t reseed, mctsnc_result *results) {
    int rc = mctsnc_search_batch_device(h, batch, boards, extras, turns, steps, reseed, nullptr, nullptr);
    if (rc) return rc;
    return mctsnc_finish_batch_device(h, batch, nullptr, results, nullptr);
}

// per-node fields of Gomoku trees in the reference's formats (see mctsnc_export)
static int export_nodes_gomoku(mctsnc_handle *h, const std::vector<TreeState> &st, long long g0, int field, void *dst,
                               long long max_nodes) {
    constexpr int A = gomoku::A;
    const int T = h->cfg.n_trees;
    const long long cap = h->cfg.node_capacity;
    const int extra = h->cfg.extra_info_memory < 1 ? 1 : h->cfg.extra_info_memory;
    std::vector<int4> rec;
    std::vector<unsigned> brd;
    std::vector<int> par;
    for (int t = 0; t < T; t++) {
        long long n = st[t].size < max_nodes ? st[t].size : max_nodes;
        if (n > cap) n = cap;
        rec.resize((size_t)n);
        CUDA_TRY(cudaMemcpy(rec.data(), h->rec + (g0 + t) * cap, sizeof(int4) * n, cudaMemcpyDeviceToHost));
        if (field == MCTSNC_F_TREES) {
            par.resize((size_t)n);
            CUDA_TRY(cudaMemcpy(par.data(), h->parent + (g0 + t) * cap, sizeof(int) * n, cudaMemcpyDeviceToHost));
        }
        if (field == MCTSNC_F_TREES || field == MCTSNC_F_BOARDS) {
            brd.resize((size_t)n * 16);
            CUDA_TRY(cudaMemcpy(brd.data(), h->gboard + (g0 + t) * cap * 16, sizeof(unsigned) * 16 * n, cudaMemcpyDeviceToHost));
        }
        for (long long i = 0; i < max_nodes; i++) {
            const bool valid = i < n;
            const int4 r = valid ? rec[(size_t)i] : make_int4(0, 0, -1, 0);
            const long long o = (long long)t * max_nodes + i;
            const unsigned *b = valid && !brd.empty() ? &brd[(size_t)i * 16] : nullptr;
            switch (field) {
            case MCTSNC_F_TREES: {
                int32_t *row = (int32_t *)dst + o * (1 + A);
                row[0] = valid ? par[(size_t)i] : -1;
                const int n_children = r.w & gomoku::G_NCHILD_MASK;
                int rank = 0;
                for (int a = 0; a < A; a++) {
                    const bool empty = valid && !(((b[a >> 5] | b[8 + (a >> 5)]) >> (a & 31)) & 1u);
                    row[1 + a] = (empty && rank < n_children) ? r.z + rank : -1;
                    rank += empty;
                }
                break;
            }
            case MCTSNC_F_DEPTHS: ((int16_t *)dst)[o] = valid ? (int16_t)meta_depth(r.w) : 0; break;
            case MCTSNC_F_TURNS: ((int8_t *)dst)[o] = valid ? (int8_t)gomoku::g_turn(r.w) : 0; break;
            case MCTSNC_F_LEAVES: ((uint8_t *)dst)[o] = valid ? ((r.w & gomoku::G_NCHILD_MASK) == 0) : 0; break;
            case MCTSNC_F_TERMINALS: ((uint8_t *)dst)[o] = valid ? ((r.w & gomoku::G_TERMINAL) != 0) : 0; break;
            case MCTSNC_F_OUTCOMES: ((int8_t *)dst)[o] = valid ? (int8_t)gomoku::g_outcome(r.w) : 0; break;
            case MCTSNC_F_NS: ((int32_t *)dst)[o] = valid ? r.x : 0; break;
            case MCTSNC_F_NS_WINS: ((int32_t *)dst)[o] = valid ? r.y : 0; break;
            case MCTSNC_F_BOARDS: {
                int8_t *bo = (int8_t *)dst + o * A;
                for (int a = 0; a < A; a++)
                    bo[a] = !valid ? 0 : (((b[8 + (a >> 5)] >> (a & 31)) & 1u) ? 1 : (((b[a >> 5] >> (a & 31)) & 1u) ? -1 : 0));
                break;
            }
            case MCTSNC_F_EXTRA_INFOS: memset((int8_t *)dst + o * extra, 0, extra); break;
            }
        }
    }
    return 0;
}

extern "C" int mctsnc_export(mctsnc_handle *h, int32_t search, int32_t field, void *dst, int64_t max_nodes) {
    if (!h || !dst || search < 0 || search >= h->cfg.max_batch) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    CUDA_TRY(cudaDeviceSynchronize());
    const int T = h->cfg.n_trees, A = h->A;
    const long long cap = h->cfg.node_capacity;
    const long long g0 = (long long)search * T;
    std::vector<TreeState> st(T);
    CUDA_TRY(cudaMemcpy(st.data(), h->state + g0, sizeof(TreeState) * T, cudaMemcpyDeviceToHost));
    switch (field) {
    case MCTSNC_F_SIZES:
        for (int t = 0; t < T; t++) ((int32_t *)dst)[t] = st[t].size;
        return 0;
    case MCTSNC_F_NODES_SELECTED:
        for (int t = 0; t < T; t++) ((int32_t *)dst)[t] = st[t].selected;
        return 0;
    case MCTSNC_F_PLAYOUT_OUTCOMES:
        for (int t = 0; t < T; t++) {
            ((int32_t *)dst)[2 * t] = st[t].out_neg;
            ((int32_t *)dst)[2 * t + 1] = st[t].out_pos;
        }
        return 0;
    case MCTSNC_F_SELECTED_PATHS: {
        std::vector<int> paths((size_t)T * PATH_CAP);
        CUDA_TRY(cudaMemcpy(paths.data(), h->paths + g0 * PATH_CAP, sizeof(int) * paths.size(), cudaMemcpyDeviceToHost));
        int32_t *o = (int32_t *)dst;
        memset(o, 0, sizeof(int32_t) * T * (MAX_TREE_DEPTH + 2));
        for (int t = 0; t < T; t++) {
            for (int e = 0; e < st[t].path_len && e < PATH_CAP; e++) o[(long long)t * (MAX_TREE_DEPTH + 2) + e] = paths[(size_t)t * PATH_CAP + e];
            o[(long long)t * (MAX_TREE_DEPTH + 2) + MAX_TREE_DEPTH + 1] = st[t].path_len;
        }
        return 0;
    }
    case MCTSNC_F_ACTIONS_EXPANDED:
        CUDA_TRY(cudaMemcpy(dst, h->actions_expanded + g0 * (A + 2), sizeof(short) * T * (A + 2), cudaMemcpyDeviceToHost));
        return 0;
    case MCTSNC_F_PLAYOUT_OUTCOMES_CHILDREN:
        CUDA_TRY(cudaMemcpy(dst, h->child_out + g0 * A * 2, sizeof(int) * T * A * 2, cudaMemcpyDeviceToHost));
        return 0;
    default:
        break;
    }
    if (field < 0 || field > MCTSNC_F_EXTRA_INFOS || max_nodes < 1) return MCTSNC_E_BAD_ARGUMENT;
    if (is_gomoku(h->cfg)) return export_nodes_gomoku(h, st, g0, field, dst, max_nodes);
    const int cells = h->cfg.board_rows * h->cfg.board_cols;
    const int extra = h->cfg.extra_info_memory;
    std::vector<int4> rec;
    std::vector<ulonglong2> brd;
    std::vector<int> par;
    for (int t = 0; t < T; t++) {
        long long n = st[t].size < max_nodes ? st[t].size : max_nodes;
        if (n > cap) n = cap;
        rec.resize((size_t)n);
        CUDA_TRY(cudaMemcpy(rec.data(), h->rec + (g0 + t) * cap, sizeof(int4) * n, cudaMemcpyDeviceToHost));
        if (field == MCTSNC_F_TREES) {
            par.resize((size_t)n);
            CUDA_TRY(cudaMemcpy(par.data(), h->parent + (g0 + t) * cap, sizeof(int) * n, cudaMemcpyDeviceToHost));
        }
        if (field == MCTSNC_F_BOARDS || field == MCTSNC_F_EXTRA_INFOS) {
            brd.resize((size_t)n);
            CUDA_TRY(cudaMemcpy(brd.data(), h->board + (g0 + t) * cap, sizeof(ulonglong2) * n, cudaMemcpyDeviceToHost));
        }
        for (long long i = 0; i < max_nodes; i++) {
            const bool valid = i < n;
            const int4 r = valid ? rec[(size_t)i] : make_int4(0, 0, -1, 0);
            const long long o = (long long)t * max_nodes + i;
            switch (field) {
            case MCTSNC_F_TREES: {
                int32_t *row = (int32_t *)dst + o * (1 + A);
                row[0] = valid ? par[(size_t)i] : -1;
                const unsigned mask = r.w & 0x7F;
                int k = 0;
                for (int a = 0; a < A; a++) row[1 + a] = (valid && ((mask >> a) & 1u)) ? r.z + k++ : -1;
                break;
            }
            case MCTSNC_F_DEPTHS: ((int16_t *)dst)[o] = valid ? (int16_t)meta_depth(r.w) : 0; break;
            case MCTSNC_F_TURNS: ((int8_t *)dst)[o] = valid ? (int8_t)meta_turn(r.w) : 0; break;
            case MCTSNC_F_LEAVES: ((uint8_t *)dst)[o] = valid ? ((r.w & 0x7F) == 0) : 0; break;
            case MCTSNC_F_TERMINALS: ((uint8_t *)dst)[o] = valid ? ((r.w & META_TERMINAL) != 0) : 0; break;
            case MCTSNC_F_OUTCOMES: ((int8_t *)dst)[o] = valid ? (int8_t)meta_outcome(r.w) : 0; break;
            case MCTSNC_F_NS: ((int32_t *)dst)[o] = valid ? r.x : 0; break;
            case MCTSNC_F_NS_WINS: ((int32_t *)dst)[o] = valid ? r.y : 0; break;
            case MCTSNC_F_BOARDS: {
                int8_t *bo = (int8_t *)dst + o * cells;
                memset(bo, 0, cells);
                if (valid)
                    for (int j = 0; j < c4::COLS; j++)
                        for (int hgt = 0; hgt < c4::ROWS; hgt++) {
                            const int bit = 7 * j + hgt;
                            const int v = ((brd[(size_t)i].y >> bit) & 1ULL) ? 1 : (((brd[(size_t)i].x >> bit) & 1ULL) ? -1 : 0);
                            bo[(c4::ROWS - 1 - hgt) * c4::COLS + j] = (int8_t)v;
                        }
                break;
            }
            case MCTSNC_F_EXTRA_INFOS: {
                int8_t *eo = (int8_t *)dst + o * extra;
                memset(eo, 0, extra);
                if (valid) {
                    const unsigned long long all = brd[(size_t)i].x | brd[(size_t)i].y;
                    for (int j = 0; j < c4::COLS; j++) eo[j] = (int8_t)__builtin_popcountll((all >> (7 * j)) & 0x3FULL);
                }
                break;
            }
            }
        }
    }
    return 0;
}

extern "C" int mctsnc_export_rng(mctsnc_handle *h, int32_t search, int32_t which, uint64_t *dst, int64_t n) {
    if (!h || !dst || search < 0 || search >= h->cfg.max_batch || n < 0) return MCTSNC_E_BAD_ARGUMENT;
    CUDA_TRY(cudaSetDevice(h->cfg.device));
    CUDA_TRY(cudaDeviceSynchronize());
    if (which == 0) {
        if (n > h->rng_per_search) return MCTSNC_E_BAD_ARGUMENT;
        CUDA_TRY(cudaMemcpy(dst, h->rng_playout + (long long)search * h->rng_per_search, sizeof(ulonglong2) * n, cudaMemcpyDeviceToHost));
    } else {
        if (!is_ocp(h->cfg) || n > h->cfg.n_trees) return MCTSNC_E_BAD_ARGUMENT;
        CUDA_TRY(cudaMemcpy(dst, h->rng_expand + (long long)search * h->cfg.n_trees, sizeof(ulonglong2) * n, cudaMemcpyDeviceToHost));
    }
    return 0;
}

extern "C" int mctsnc_query(mctsnc_handle *h, int32_t *threads_per_tree, int32_t *blocks_per_sm, int32_t *sm_count,
                            int64_t *bytes_allocated) {
    if (!h) return MCTSNC_E_BAD_ARGUMENT;
    if (threads_per_tree) *threads_per_tree = h->threads;
    if (blocks_per_sm) *blocks_per_sm = h->blocks_per_sm;
    if (sm_count) *sm_count = h->sm_count;
    if (bytes_allocated) *bytes_allocated = h->bytes;
    return 0;
}

extern "C" int mctsnc_trace_slices(mctsnc_handle *h, int32_t max_records) {
    if (!h || max_records < 0) return MCTSNC_E_BAD_ARGUMENT;
    cudaFree(h->trace);
    cudaFree(h->trace_count);
    h->trace = nullptr;
    h->trace_count = nullptr;
    h->trace_cap = 0;
    if (max_records == 0) return 0;
    int rc = dev_alloc(h, &h->trace, 4LL * max_records);
    if (!rc) rc = dev_alloc(h, &h->trace_count, 1);
    if (rc) return rc;
    CUDA_TRY(cudaMemset(h->trace_count, 0, sizeof(int)));
    h->trace_cap = max_records;
    return 0;
}

extern "C" int mctsnc_read_slices(mctsnc_handle *h, int64_t *dst, int32_t max_records, int32_t *n_records) {
    if (!h || !n_records || (max_records > 0 && !dst)) return MCTSNC_E_BAD_ARGUMENT;
    *n_records = 0;
    if (!h->trace) return 0;
    int n = 0;
    CUDA_TRY(cudaMemcpy(&n, h->trace_count, sizeof(int), cudaMemcpyDeviceToHost));
    if (n > h->trace_cap) n = h->trace_cap;
    if (n > max_records) n = max_records;
    if (n > 0) CUDA_TRY(cudaMemcpy(dst, h->trace, sizeof(long long) * 4 * n, cudaMemcpyDeviceToHost));
    *n_records = n;
    return 0;
}

extern "C" const char *mctsnc_error_string(int code) {
    switch (code) {
    case 0: return "success";
    case MCTSNC_E_BAD_ARGUMENT: return "mctsnc: bad argument";
    case MCTSNC_E_UNSUPPORTED: return "mctsnc: game or shape not supported by this build";
    case MCTSNC_E_NO_MEMORY: return "mctsnc: out of memory";
    case MCTSNC_E_BAD_ROOT: return "mctsnc: root board and extra_info do not describe a reachable, unfinished position";
    case MCTSNC_E_CAPACITY: return "mctsnc: batch or step count beyond the capacity of the handle";
    case MCTSNC_E_NO_DEVICE: return "mctsnc: no CUDA device";
    default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "mctsnc: unknown error";
}

// ===================================================================================================================
// mctsnc_search_c4_static: one Connect-4 search that allocates nothing.
//
// Every other entry point works on a handle whose pools come from cudaMalloc in mctsnc_create.  Some callers cannot do
// that: code that runs while a framework's caching allocator owns the whole device, services that forbid allocation
// after start-up so that a search can never fail for lack of memory, plug-ins that are handed a stream and two buffers
// and nothing else.  For them the tree pools, the random streams and the per-tree bookkeeping of this variant live in
// one file-scope device array of fixed size (every device that loads the library carries it until the process exits),
// so the limits below are modest.
//
// The array's name is only a host-side stand-in for the device object, not a device address: the first call on a device
// (with that device current) asks the runtime for the address with cudaGetSymbolAddress and every launch gets that
// pointer.  That first call also fills the cache of seeded streams; it synchronises, so it has to come before any
// stream capture.  All calls share the one array and it keeps what the last call left: what has to start from zero is
// cleared on the caller's stream at the start of every call, and two calls whose work overlaps on the GPU (different
// streams, different host threads) would race on it -- run them one after the other.  The host-side statics (address
// per device, stream cache, staging buffer) are guarded by a mutex.
namespace {
namespace fixed {

constexpr int MAX_TREES = MCTSNC_STATIC_MAX_TREES;
constexpr int MAX_PLAYOUTS = MCTSNC_STATIC_MAX_PLAYOUTS;
constexpr int MAX_STEPS = MCTSNC_STATIC_MAX_STEPS;
constexpr int A = c4::A;
constexpr long long CAP = (long long)MAX_STEPS * A + 1 + A;   // nodes per tree
constexpr int MAX_STREAMS = MAX_TREES * A * MAX_PLAYOUTS;
constexpr int MAX_DEVICES = 64;

struct Scratch {
    int4 rec[MAX_TREES * CAP];
    ulonglong2 board[MAX_TREES * CAP];
    ulonglong2 rng[MAX_STREAMS];
    ulonglong2 rng_base[MAX_STREAMS];
    ulonglong2 rng_expand[MAX_TREES];
    ulonglong2 rng_expand_base[MAX_TREES];
    ulonglong2 root_board[1];
    long long sums[3 * A];
    DevResult dres[1];
    TreeState state[MAX_TREES];
    int parent[MAX_TREES * CAP];
    int paths[MAX_TREES * PATH_CAP];
    int child_out[MAX_TREES * A * 2];
    short actions_expanded[MAX_TREES * (A + 2)];
    unsigned char flags[2 * A];
    signed char root_turn[16];
};

// the figure quoted in include/mctsnc_b200.h ("about 0.75 MB")
static_assert(sizeof(Scratch) > 700 * 1024 && sizeof(Scratch) < 800 * 1024, "update the size quoted in the header");

static __device__ __align__(256) unsigned char g_static_scratch[sizeof(Scratch)];

struct DeviceSetup {
    Scratch *ptr = nullptr;       // device address of g_static_scratch on this device
    bool streams_cached = false;  // rng_base / rng_expand_base hold the streams of the key below
    unsigned long long seed = 0;
    int n_trees = 0, n_playouts = 0, ocp = 0;
};
DeviceSetup g_setup[MAX_DEVICES];
ulonglong2 g_host_streams[MAX_STREAMS];   // staging for the seeded streams (static: no host allocation either)
std::mutex g_setup_mutex;                 // the two objects above are shared by all devices and all host threads

// the root arrives as kernel arguments (by value): no host memory is read after the call has returned
__global__ void set_root_kernel(ulonglong2 *root_board, signed char *root_turn, ulonglong2 root, int turn) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        root_board[0] = root;
        root_turn[0] = (signed char)turn;
    }
}

__global__ void copy_streams_kernel(ulonglong2 *dst, const ulonglong2 *src, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// [root_ns | actions_ns | actions_ns_wins] are already in `out`; append best action, win flag, n, n_wins
__global__ void append_best_kernel(const DevResult *dres, long long *out, int A_) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        out[3 * A_ + 0] = dres->best_action;
        out[3 * A_ + 1] = dres->best_win_flag;
        out[3 * A_ + 2] = dres->best_n;
        out[3 * A_ + 3] = dres->best_n_wins;
    }
}

}  // namespace fixed
}  // namespace

extern "C" int mctsnc_search_c4_static(const int8_t *board, const int8_t *extra_info, int32_t turn, int32_t variant,
                                       int32_t n_trees, int32_t n_playouts, int64_t steps, float ucb_c, uint64_t seed,
                                       int64_t *out_device, void *stream) {
    using namespace fixed;
    if (!board || !out_device || (turn != 1 && turn != -1) || variant < 0 || variant > 3 || n_trees < 1 || n_playouts < 1 ||
        (n_playouts & (n_playouts - 1)) != 0 || steps < 0 || !(ucb_c >= 0.f))
        return MCTSNC_E_BAD_ARGUMENT;
    if (n_trees > MAX_TREES || n_playouts > MAX_PLAYOUTS || steps > MAX_STEPS) return MCTSNC_E_CAPACITY;
    int device = -1;
    CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= MAX_DEVICES) return MCTSNC_E_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    ulonglong2 root;
    int rc = c4_encode_root(board, extra_info, &root);
    if (rc) return rc;
    // the set-up below touches host-side state shared by every device and thread: one caller at a time
    std::unique_lock<std::mutex> setup_lock(g_setup_mutex);
    DeviceSetup &su = g_setup[device];
    if (!su.ptr) {
        // once per device, with that device current: the device address behind the symbol
        void *p = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        su.ptr = reinterpret_cast<Scratch *>(p);
        su.streams_cached = false;
    }
    Scratch *sc = su.ptr;
    const bool ocp = variant == MCTSNC_OCP_THRIFTY || variant == MCTSNC_OCP_PRODIGAL;
    const int per_tree = ocp ? n_playouts : A * n_playouts;
    const int n_streams = n_trees * per_tree;
    if (!su.streams_cached || su.seed != seed || su.n_trees != n_trees || su.n_playouts != n_playouts || su.ocp != (int)ocp) {
        // seeded streams of this configuration (numba's create_xoroshiro128p_states): computed on the host into a
        // static buffer and kept on the device for the calls to come
        su.streams_cached = false;
        CUDA_TRY(cudaStreamSynchronize(s));  // the staging buffer is reused: nothing may still be reading it
        make_streams(seed, 0, n_streams, 1, g_host_streams);
        CUDA_TRY(cudaMemcpyAsync(sc->rng_base, g_host_streams, sizeof(ulonglong2) * n_streams, cudaMemcpyHostToDevice, s));
        CUDA_TRY(cudaStreamSynchronize(s));
        if (ocp) {
            const int tpb_e1 = 64;  // Connect 4: min(max(pow2(42), pow2(7)), 512), src/mctsnc.py:360-365
            make_streams(seed, 0, n_trees, tpb_e1, g_host_streams);
            CUDA_TRY(cudaMemcpyAsync(sc->rng_expand_base, g_host_streams, sizeof(ulonglong2) * n_trees, cudaMemcpyHostToDevice, s));
            CUDA_TRY(cudaStreamSynchronize(s));
        }
        su.seed = seed;
        su.n_trees = n_trees;
        su.n_playouts = n_playouts;
        su.ocp = (int)ocp;
        su.streams_cached = true;
    }
    setup_lock.unlock();
    // what has to start from zero, and the root
    CUDA_TRY(cudaMemsetAsync(sc->state, 0, sizeof(sc->state), s));
    CUDA_TRY(cudaMemsetAsync(sc->child_out, 0, sizeof(sc->child_out), s));
    CUDA_TRY(cudaMemsetAsync(sc->actions_expanded, 0, sizeof(sc->actions_expanded), s));
    set_root_kernel<<<1, 32, 0, s>>>(sc->root_board, sc->root_turn, root, turn);
    copy_streams_kernel<<<32, 256, 0, s>>>(sc->rng, sc->rng_base, n_streams);
    if (ocp) copy_streams_kernel<<<1, 32, 0, s>>>(sc->rng_expand, sc->rng_expand_base, n_trees);
    SearchParams p;
    p.rec = sc->rec;
    p.board = sc->board;
    p.parent = sc->parent;
    p.state = sc->state;
    p.paths = sc->paths;
    p.actions_expanded = sc->actions_expanded;
    p.child_out = sc->child_out;
    p.rng_playout = sc->rng;
    p.rng_expand = sc->rng_expand;
    p.root_board = sc->root_board;
    p.root_turn = sc->root_turn;
    p.cap = CAP;
    p.node_limit = CAP;
    p.n_trees = n_trees;
    p.n_playouts = n_playouts;
    p.log2_playouts = 0;
    while ((1 << p.log2_playouts) < n_playouts) p.log2_playouts++;
    p.n_actions = A;
    p.variant = variant;
    p.steps = (int)steps;
    p.first = 1;
    p.ucb_c = ucb_c;
    p.queue = nullptr;
    p.ring = nullptr;
    p.remaining = nullptr;
    p.ring_cap = 0;
    p.chunk = 0;
    p.trace = nullptr;
    p.trace_count = nullptr;
    p.trace_cap = 0;
    p.ms_per_cycle = 0.f;
    p.cache_nodes = 0;
    const size_t dyn_smem = sizeof(ulonglong2) * (size_t)per_tree;   // <= 28 KB: below the 48 KB that need an opt-in
    if (ocp) c4::search_kernel<true><<<n_trees, 256, dyn_smem, s>>>(p);
    else c4::search_kernel<false><<<n_trees, 256, dyn_smem, s>>>(p);
    CUDA_TRY(cudaGetLastError());
    long long *out = reinterpret_cast<long long *>(out_device);
    reduce_over_trees_kernel<<<1, 256, 0, s>>>(sc->rec, sc->state, CAP, n_trees, A, out, sc->flags, sc->dres);
    const bool thrifty = variant == MCTSNC_OCP_THRIFTY || variant == MCTSNC_ACP_THRIFTY;
    reduce_over_actions_kernel<<<1, 8, 0, s>>>(out, sc->flags, A, 8, thrifty ? 1 : 0, sc->dres);
    append_best_kernel<<<1, 32, 0, s>>>(sc->dres, out, A);
    return (int)cudaGetLastError();
}
