// Data layout shared by the search kernels and the host side of libmctsnc_b200.
//
// One search grows n_trees independent trees; a batch holds `batch` searches.  Tree g = search * n_trees + tree owns
// the node range [g * cap, (g + 1) * cap) of three structure-of-arrays pools:
//
//   rec[node]    int4  { ns, ns_wins, first_child, meta }    16 B  -- everything the UCB descent needs
//   board[node]  16 B  game-specific packed position (Connect-4: two 64-bit bitboards)
//   parent[node] int32                                       -- only read when a tree is exported
//
// The children of a node are created together and occupy consecutive slots (the reference assigns
// child = size_so_far + shift in ascending action order, src/mctsnc.py:1426-1429 and :1450), so a node stores only
// the first child and the set of expanded actions; one 16-byte load per child then yields its statistics AND its own
// child pointer, which makes the descent one dependent memory access per level.
//
// meta:  bits 0..6   expanded-action set (Connect-4; games with more actions keep the set in a side array)
//        bit  7      terminal          (trees_terminals)
//        bits 8..9   outcome + 1, 3 = game ongoing (trees_outcomes)
//        bit  10     1 if the player to move is +1 (trees_turns)
//        bits 16..31 depth             (trees_depths)
// A node is a leaf (trees_leaves) while its expanded-action set is empty.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mctsnc {

constexpr int META_TERMINAL = 1 << 7;
constexpr int META_OUTCOME_SHIFT = 8;
constexpr int META_TURN_POS = 1 << 10;
constexpr int META_DEPTH_SHIFT = 16;

constexpr int MODE_ALL_CHILDREN = -2;  // trees_actions_expanded[ti, -2] of the ACP variants
constexpr int MODE_TERMINAL = -1;      // the selected node is terminal
constexpr int MODE_TREE_FULL = -3;     // no room for any child
constexpr int MODE_DONE = -4;          // inside a kernel: the steps of the launch are done

constexpr unsigned STATUS_TREE_FULL = 1u;
constexpr unsigned STATUS_UB_DRAW = 2u;
constexpr unsigned STATUS_INTERNAL = 4u;

constexpr int PATH_CAP = 256;  // longest root-to-leaf path kept per tree (Connect-4: 43, Gomoku: 226)

__host__ __device__ __forceinline__ int meta_outcome(int meta) { return ((meta >> META_OUTCOME_SHIFT) & 3) - 1; }
__host__ __device__ __forceinline__ int meta_turn(int meta) { return (meta & META_TURN_POS) ? 1 : -1; }
__host__ __device__ __forceinline__ int meta_depth(int meta) { return (meta >> META_DEPTH_SHIFT) & 0xFFFF; }
__host__ __device__ __forceinline__ int make_meta(int mask, bool terminal, int outcome, int turn, int depth) {
    return mask | (terminal ? META_TERMINAL : 0) | ((outcome + 1) << META_OUTCOME_SHIFT) |
           (turn > 0 ? META_TURN_POS : 0) | (depth << META_DEPTH_SHIFT);
}

// Per-tree bookkeeping that outlives a launch (a time-limited search is a sequence of launches) and that the export
// functions read: the "last step" arrays of the reference (trees_nodes_selected, trees_selected_paths,
// trees_actions_expanded, trees_playout_outcomes[_children]) and the library's own counters.
struct TreeState {
    int size;            // trees_sizes
    int selected;        // trees_nodes_selected
    int path_len;        // trees_selected_paths[ti, -1]
    int out_neg;         // trees_playout_outcomes[ti, 0]
    int out_pos;         // trees_playout_outcomes[ti, 1]
    unsigned status;
    unsigned long long plies;
    unsigned long long ub_draws;
    float us_per_step;   // work queue: smoothed time per step of the tree's slices in the current launch (microseconds)
    // time this tree's block spent in the four stages of its steps since the search began, in milliseconds at the nominal
    // SM clock (cycle counter of the SM the block ran on): select, expand, playouts, backup.  The reference times the same
    // stages with host clocks around its launches (src/mctsnc.py:606-686).
    float stage_ms[4];
    int reserved;
};

// Work queue of a batched launch.  A tree's search is cut into slices of `chunk` steps; the blocks of a persistent grid
// take a tree from the queue, run one slice from the state the previous slice left in global memory, and put the tree
// back while it has steps left.  A tree is sequential, so a launch cannot end before its slowest tree (the one whose
// games are longest) has done all its steps: the queue therefore serves the trees with the most work left first
// (longest remaining processing time first, the rule that minimises the makespan of preemptible jobs on identical
// machines), with the time left estimated as steps left x time per step of the slice just run.  QUEUE_LEVELS rings,
// one per band of time left; a pop takes from the highest ring that holds a tree.
//
// Each ring is a bounded multi-producer multi-consumer queue with a sequence number per cell (cell i is free for the
// push with ticket t when seq == t, holds the data of that push when seq == t + 1, and is handed to ticket t + cap by
// the pop).  `nonempty` has one bit per ring, set after a push and cleared by a pop that found the ring empty and, after
// clearing, still sees it empty.  Every loop is bounded and no call waits for another block: a pop that finds nothing
// (or gives up) returns -1 and the block leaves, which is safe because a tree is always either in a ring or held by a
// block that will publish it and pop again.
constexpr int QUEUE_LEVELS = 64;
constexpr float QUEUE_LEVELS_PER_OCTAVE = 6.f;  // bands are logarithmic: the estimate's error grows with the time left
struct QueueCell {
    int seq;
    int tree;
};
struct WorkQueue {
    int head;
    int pad0[31];
    int tail;
    int pad1[31];
};
struct WorkQueues {
    WorkQueue level[QUEUE_LEVELS];
    unsigned long long nonempty;
    int longest_us;  // longest estimate so far of a whole search's time (microseconds); the top band
    int pad[29];
};

constexpr int QUEUE_RETRIES = 1 << 16;  // attempts of a push or pop under contention before it reports failure

#if defined(__CUDACC__)
__device__ __forceinline__ bool ring_push(WorkQueue *q, QueueCell *ring, int cap, int tree) {
    for (int attempt = 0; attempt < QUEUE_RETRIES; attempt++) {
        const int pos = *(volatile int *)&q->tail;
        QueueCell *cell = ring + (pos % cap);
        const int dif = *(volatile int *)&cell->seq - pos;
        if (dif == 0) {
            if (atomicCAS(&q->tail, pos, pos + 1) == pos) {
                *(volatile int *)&cell->tree = tree;
                __threadfence();
                *(volatile int *)&cell->seq = pos + 1;
                return true;
            }
        } else if (dif < 0) {
            return false;  // ring full: cannot happen while cap >= number of trees
        }
    }
    return false;
}

// -1: nothing published (or QUEUE_RETRIES lost races in a row)
__device__ __forceinline__ int ring_pop(WorkQueue *q, QueueCell *ring, int cap) {
    for (int attempt = 0; attempt < QUEUE_RETRIES; attempt++) {
        const int pos = *(volatile int *)&q->head;
        QueueCell *cell = ring + (pos % cap);
        const int dif = *(volatile int *)&cell->seq - (pos + 1);
        if (dif == 0) {
            if (atomicCAS(&q->head, pos, pos + 1) == pos) {
                __threadfence();
                const int tree = *(volatile int *)&cell->tree;
                __threadfence();
                *(volatile int *)&cell->seq = pos + cap;
                return tree;
            }
        } else if (dif < 0) {
            // no ticket beyond the head: empty.  Otherwise a push holds the ticket and is about to publish: look again.
            if (*(volatile int *)&q->tail - pos <= 0) return -1;
        }
    }
    return -1;
}

// the caller made the tree's state visible (block barrier after the writes, then this thread's fence) before the push
__device__ __forceinline__ bool queue_push(WorkQueues *q, QueueCell *rings, int cap, int level, int tree) {
    if (!ring_push(&q->level[level], rings + (long long)level * cap, cap, tree)) return false;
    __threadfence();
    atomicOr(&q->nonempty, 1ULL << level);
    return true;
}

__device__ __forceinline__ int queue_pop(WorkQueues *q, QueueCell *rings, int cap) {
    for (int attempt = 0; attempt < 8 * QUEUE_LEVELS; attempt++) {
        const unsigned long long m = *(volatile unsigned long long *)&q->nonempty;
        if (m == 0) return -1;
        const int level = 63 - __clzll((long long)m);
        WorkQueue *r = &q->level[level];
        const int tree = ring_pop(r, rings + (long long)level * cap, cap);
        if (tree >= 0) return tree;
        // the ring was empty: clear its bit, then look once more; a push that slipped in between either set the bit after
        // this clear or is seen by the second look (both sides go through read-modify-write operations and a fence)
        atomicAnd(&q->nonempty, ~(1ULL << level));
        __threadfence();
        if (atomicAdd(&r->tail, 0) - atomicAdd(&r->head, 0) > 0) atomicOr(&q->nonempty, 1ULL << level);
    }
    return -1;
}
#endif

struct SearchParams {
    int4 *rec;
    ulonglong2 *board;
    int *parent;
    TreeState *state;        // [trees]
    int *paths;              // [trees][PATH_CAP]
    short *actions_expanded; // [trees][A + 2], reference layout of the handle's variant
    int *child_out;          // [trees][A][2]  trees_playout_outcomes_children
    ulonglong2 *rng_playout; // ACP: [trees][A][P], OCP: [trees][P]
    ulonglong2 *rng_expand;  // OCP: [trees]
    const ulonglong2 *root_board;  // [batch]
    const signed char *root_turn;  // [batch]
    long long cap;           // nodes allocated per tree
    long long node_limit;    // min(max_tree_size, cap): a tree never grows beyond it
    int n_trees;             // trees per search (this handle)
    int n_playouts;
    int log2_playouts;
    int n_actions;
    int variant;
    int steps;               // steps to carry out in this launch
    int first;               // 1: reset the trees to the roots first (the reference's _reset)
    float ucb_c;
    // batched launches through the work queue; queue == nullptr: block b runs all `steps` of tree b
    WorkQueues *queue;
    QueueCell *ring;         // [QUEUE_LEVELS][ring_cap]
    int *remaining;          // [trees] steps of this launch a tree still has to do
    int ring_cap;
    int chunk;               // steps per slice
    // optional record of every slice of a queued launch (nullptr: none): 4 words per slice -- tree, start and end in
    // nanoseconds of %globaltimer, (SM id << 32) | steps
    long long *trace;
    int *trace_count;
    int trace_cap;
    float ms_per_cycle;      // 1 / (nominal SM clock in kHz): converts cycle counts into the stage times of TreeState
    int cache_nodes;         // cluster kernel: node records of a tree (the first ones) kept in the first block's shared memory
};

}  // namespace mctsnc
