// Decoupled-UCT (DUCT) select and backup for simultaneous-move games: two players, A actions each (A <= 16), a child
// per joint action.  NO COUNTERPART IN THE REFERENCE: src/puct holds only the single-agent PUCT select; the benchmark
// configuration "DUCT 2 x 8 joint actions" names a variant the reference does not implement, so the semantics below are
// this library's own (stated in include/duct_b200.h and restated on the CPU in oracle/duct_oracle.py) and parity is
// unpinned by construction.  The conventions of the PUCT select are kept where they apply: one warp per traversal,
// grid = trees, block = warps * 32, path entries (node << 8) | slot, packed results
// reason << 25 | kind << 22 | slot << 14 | node, virtual loss claimed on the way down and returned by the backup.
//
// One level costs one memory round trip: lane l holds the statistics of action l % 16 of player l / 16 and, next to
// them, its share of the node's A*A child ids, all requested together with the node's terminal flag; the two arg-maxes
// are warp-reduce instructions over the half-warps; the claims are fire-and-forget atomics; the winner's child id is
// already in a register, so the next level's loads can leave at once.
#include <cuda_runtime.h>
#include <stdint.h>

namespace duct {

constexpr unsigned FULL = 0xFFFFFFFFu;
constexpr int MAX_ACTIONS = 16, NODE_LIMIT = 16384;
constexpr int KIND_SHIFT = 22, SLOT_SHIFT = 14, REASON_SHIFT = 25;
constexpr int CHILD_NONE = -1, CHILD_CLAIMED = -2;
enum Kind { INVALID = 0, EXPAND = 1, TERMINAL = 2, DEPTH_LIMIT = 3, BUSY = 4 };
enum Reason { R_UNSET = 0, R_OK_EXPAND = 1, R_OK_TERMINAL = 2, R_OK_DEPTH_LIMIT = 3, R_BUSY_EXPAND_INFLIGHT = 4,
              R_INVALID_SHAPE = 10, R_INVALID_CHILD_OOB = 15 };
constexpr int CHILD_SLOTS = MAX_ACTIONS * MAX_ACTIONS / 32;  // child ids a lane may hold
constexpr int MAX_EVALUATIONS = 3;  // arg-max evaluations of a player at one node before its pick is claimed regardless

__device__ __forceinline__ int pack(int kind, int node, int slot, int reason) {
    return (reason << REASON_SHIFT) | (kind << KIND_SHIFT) | (slot << SLOT_SHIFT) | node;
}

__device__ __forceinline__ unsigned ordered(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// score of one action of one player; every operation rounds once, in this order (the CPU restatement does the same)
__device__ __forceinline__ float score(float cpuct, float prior, float w, int n, int inflight, int virtual_loss, float sqrt_total) {
    const int n_eff = n + virtual_loss * inflight;
    const float w_eff = __fsub_rn(w, (float)(virtual_loss * inflight));  // a traversal in flight counts as a loss
    const float q = n_eff > 0 ? __fdiv_rn(w_eff, (float)n_eff) : 0.f;
    const float u = __fdiv_rn(__fmul_rn(__fmul_rn(cpuct, prior), sqrt_total), (float)(1 + n_eff));
    return __fadd_rn(q, u);
}

// gives back the claims of the first `depth` path entries of this warp
__device__ __forceinline__ void rollback(const int *path, int depth, int lane, int *node_inflight, long long stats_base, int A,
                                         int amount) {
    __syncwarp();  // the entries were written by lane 0
    for (int d = lane; d < depth; d += 32) {
        const int enc = path[d];
        const int node = enc >> 8, joint = enc & 0xFF;
        const long long s0 = stats_base + (long long)node * 2 * A;
        atomicSub(&node_inflight[s0 + joint / A], amount);
        atomicSub(&node_inflight[s0 + A + joint % A], amount);
    }
}

__global__ void select_kernel(float cpuct, int virtual_loss, int *child, const float *node_prior, const float *node_w,
                              const int *node_n, int *node_inflight, const int *node_terminal, const int *tree_nodes,
                              int *out_selected, int *out_path, int *out_len, int nodes, int A, int warps, int path_depth) {
    const int tree = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= warps) return;
    const int out = tree * warps + warp;
    int *path = out_path + (long long)out * path_depth;
    const int node_cnt = tree_nodes[tree];
    const int player = lane >> 4, action = lane & 15;
    const bool has_action = action < A;
    const unsigned half = player ? 0xFFFF0000u : 0x0000FFFFu;
    const long long stats_base = (long long)tree * nodes * 2 * A;
    const long long child_base = (long long)tree * nodes * A * A;
    const int joints = A * A;

    int node = 0, depth = 0, result = pack(INVALID, 0, 0, R_UNSET);
    if (node_cnt <= 0 || node_cnt > nodes) {
        if (lane == 0) {
            out_selected[out] = pack(INVALID, 0, 0, R_INVALID_SHAPE);
            out_len[out] = 0;
        }
        return;
    }
    for (;;) {
        // ---- everything this level needs, requested together
        const long long s = stats_base + (long long)node * 2 * A + player * A + action;
        float prior = 0.f, w = 0.f;
        int n = 0, inflight = 0;
        if (has_action) {
            prior = node_prior[s];
            w = node_w[s];
            n = node_n[s];
            inflight = *(volatile const int *)&node_inflight[s];
        }
        int kids[CHILD_SLOTS];
        const long long c0 = child_base + (long long)node * joints;
#pragma unroll
        for (int k = 0; k < CHILD_SLOTS; k++) {
            const int j = lane + 32 * k;
            kids[k] = j < joints ? *(volatile const int *)&child[c0 + j] : CHILD_NONE;
        }
        const int terminal = node_terminal[(long long)tree * nodes + node];
        if (terminal) {
            result = pack(TERMINAL, node, 0, R_OK_TERMINAL);
            break;
        }
        if (depth >= path_depth) {
            result = pack(DEPTH_LIMIT, node, 0, R_OK_DEPTH_LIMIT);
            break;
        }
        // ---- each player's arg-max over its own marginal statistics (each half-warp on its own).  The winner is claimed
        // with a compare-and-swap on the count it was scored with: if another traversal claimed it meanwhile, the counts
        // in flight are read again and the arg-max is redone, so that traversals started together spread over the
        // actions as they would one after the other; the last evaluation claims unconditionally.
        int pick = 0;
        for (int evaluation = 1;; evaluation++) {
            const int total = __reduce_add_sync(half, has_action ? n + virtual_loss * inflight : 0);
            const float sqrt_total = __fsqrt_rn((float)max(total, 1));
            const unsigned key = has_action ? ordered(score(cpuct, prior, w, n, inflight, virtual_loss, sqrt_total)) : 0u;
            const unsigned best = __reduce_max_sync(half, key);
            pick = __reduce_min_sync(half, (has_action && key == best) ? action : MAX_ACTIONS);   // lowest action on ties
            int claimed = 1;
            if (has_action && action == pick) {
                if (evaluation < MAX_EVALUATIONS) claimed = atomicCAS(&node_inflight[s], inflight, inflight + virtual_loss) == inflight;
                else atomicAdd(&node_inflight[s], virtual_loss);
            }
            if (__reduce_min_sync(half, claimed)) break;
            if (has_action) inflight = *(volatile const int *)&node_inflight[s];
        }
        const int a0 = __shfl_sync(FULL, pick, 0), a1 = __shfl_sync(FULL, pick, 16);
        const int joint = a0 * A + a1;
        if (lane == 0) path[depth] = (node << 8) | joint;
        depth++;
        int kid = CHILD_NONE;
#pragma unroll
        for (int k = 0; k < CHILD_SLOTS; k++) {
            const int v = __shfl_sync(FULL, kids[k], joint & 31);
            if ((joint >> 5) == k) kid = v;
        }
        if (kid >= 0) {
            if (kid >= node_cnt) {
                rollback(path, depth, lane, node_inflight, stats_base, A, virtual_loss);
                result = pack(INVALID, node, joint, R_INVALID_CHILD_OOB);
                depth = 0;
                break;
            }
            node = kid;
            continue;
        }
        // ---- no child yet: one traversal may expand the joint action, the others back off
        int won = 0;
        if (lane == 0) won = (kid == CHILD_NONE && atomicCAS(&child[c0 + joint], CHILD_NONE, CHILD_CLAIMED) == CHILD_NONE) ? 1 : 0;
        won = __shfl_sync(FULL, won, 0);
        if (won) {
            result = pack(EXPAND, node, joint, R_OK_EXPAND);
        } else {
            rollback(path, depth, lane, node_inflight, stats_base, A, virtual_loss);
            result = pack(BUSY, node, joint, R_BUSY_EXPAND_INFLIGHT);
            depth = 0;
        }
        break;
    }
    if (lane == 0) {
        out_selected[out] = result;
        out_len[out] = depth;
    }
}

// per path entry: both players' claims are returned, and with `values` the visit counts and value sums are updated
// (values are from player 0's point of view; player 1 receives the negative).  An EXPAND result either installs
// new_child (when given and >= 0) in the claimed slot or frees the slot again.
__global__ void backup_kernel(int virtual_loss, int *child, float *node_w, int *node_n, int *node_inflight, const int *out_selected,
                              const int *out_path, const int *out_len, const float *values, const int *new_child, int nodes, int A,
                              int warps, int path_depth) {
    const int tree = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= warps) return;
    const int out = tree * warps + warp;
    const int len = out_len[out];
    const int *path = out_path + (long long)out * path_depth;
    const long long stats_base = (long long)tree * nodes * 2 * A;
    for (int d = lane; d < len; d += 32) {
        const int enc = path[d];
        const int node = enc >> 8, joint = enc & 0xFF;
        const long long s0 = stats_base + (long long)node * 2 * A + joint / A;
        const long long s1 = stats_base + (long long)node * 2 * A + A + joint % A;
        atomicSub(&node_inflight[s0], virtual_loss);
        atomicSub(&node_inflight[s1], virtual_loss);
        if (values) {
            const float v = values[(long long)out * path_depth + d];
            atomicAdd(&node_n[s0], 1);
            atomicAdd(&node_n[s1], 1);
            atomicAdd(&node_w[s0], v);
            atomicAdd(&node_w[s1], -v);
        }
    }
    if (lane == 0) {
        const int sel = out_selected[out];
        if (((sel >> KIND_SHIFT) & 7) == EXPAND) {
            const int node = sel & (NODE_LIMIT - 1), joint = (sel >> SLOT_SHIFT) & 0xFF;
            const int kid = new_child ? new_child[out] : CHILD_NONE;
            child[((long long)tree * nodes + node) * A * A + joint] = kid >= 0 ? kid : CHILD_NONE;
        }
    }
}

}  // namespace duct

extern "C" int duct_select_launch(float cpuct, int virtual_loss, int *child, const float *node_prior, const float *node_w,
                                  const int *node_n, int *node_inflight, const int *node_terminal, const int *tree_nodes,
                                  int *out_selected, int *out_path, int *out_len, int trees, int nodes, int actions, int warps,
                                  int path_depth, void *stream) {
    if (trees <= 0 || nodes <= 0 || nodes > duct::NODE_LIMIT || actions <= 0 || actions > duct::MAX_ACTIONS || warps <= 0 ||
        warps > 32 || path_depth <= 0 || virtual_loss < 0)
        return (int)cudaErrorInvalidValue;
    duct::select_kernel<<<trees, warps * 32, 0, (cudaStream_t)stream>>>(cpuct, virtual_loss, child, node_prior, node_w, node_n,
                                                                        node_inflight, node_terminal, tree_nodes, out_selected,
                                                                        out_path, out_len, nodes, actions, warps, path_depth);
    return (int)cudaGetLastError();
}

extern "C" int duct_backup_launch(int virtual_loss, int *child, float *node_w, int *node_n, int *node_inflight,
                                  const int *out_selected, const int *out_path, const int *out_len, const float *values,
                                  const int *new_child, int trees, int nodes, int actions, int warps, int path_depth, void *stream) {
    if (trees <= 0 || nodes <= 0 || nodes > duct::NODE_LIMIT || actions <= 0 || actions > duct::MAX_ACTIONS || warps <= 0 ||
        warps > 32 || path_depth <= 0 || virtual_loss < 0)
        return (int)cudaErrorInvalidValue;
    duct::backup_kernel<<<trees, warps * 32, 0, (cudaStream_t)stream>>>(virtual_loss, child, node_w, node_n, node_inflight,
                                                                        out_selected, out_path, out_len, values, new_child, nodes,
                                                                        actions, warps, path_depth);
    return (int)cudaGetLastError();
}
