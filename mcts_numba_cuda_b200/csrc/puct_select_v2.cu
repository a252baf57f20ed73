// The two older PUCT select kernels of the reference and their backup, for trees whose virtual visits are kept per
// child NODE (node_inflight[tree, node]) instead of per edge:
//   preclaim      _select_kernel_native        src/puct/puct_gpu_v2.py:573-697   every candidate child gets +1 before it is
//                                              scored, the losers give theirs back
//   counter-CAS   _select_kernel_winner_recalc src/puct/puct_gpu_v2.py:700-840   the winner alone is claimed, by
//                                              compare-and-swap on the counter; a claim that met other visits is given
//                                              back once and the choice repeated without that edge
//   backup        _backup_kernel_native        src/puct/puct_gpu_v2.py:847-927
// Semantics followed, not the code.  Results are packed (kind << 22) | (slot << 14) | node without reason bits, a failed
// traversal rolls its path back and reports INVALID (there is no BUSY kind in this layout), path entries are
// (parent << 8) | slot.
//
// What is done differently: one traversal per small thread block (see puct_select.cu), warp reductions by redux.sync on
// an order-preserving key with a second redux for the tie-break instead of five rounds of paired shuffles, and a level
// reads child id, count, prior, value and the child's visits of every edge once, into registers (up to 8 edges a lane).
#include <cuda_runtime.h>
#include <stdint.h>

namespace puct_v2 {

constexpr unsigned FULL = 0xFFFFFFFFu;
constexpr int NODE_TERMINAL = -1;
constexpr int NODE_LIMIT = 16384, NODE_MASK = 0x3FFF, EDGE_LIMIT = 256;
constexpr int KIND_SHIFT = 22, SLOT_SHIFT = 14;
enum Kind { INVALID = 0, EXPAND = 1, TERMINAL = 2, DEPTH_LIMIT = 3 };
constexpr int PACKED_INVALID = (INVALID << KIND_SHIFT) | NODE_MASK;
constexpr int MAX_CLAIM_RETRY = 8;   // compare-and-swap attempts before the claim falls back to an atomic add (:328-347)
constexpr int MAX_RECALC = 2;        // evaluations of a level by the counter-CAS variant (:528-560)
constexpr int NO_EDGE = 0x7FFFFFFF;
constexpr int EPL = 8;               // edges per lane held in registers: 256 edges at most

__device__ __forceinline__ int pack(int kind, int node, int slot) { return (kind << KIND_SHIFT) | (slot << SLOT_SHIFT) | node; }

__device__ __forceinline__ unsigned ordered(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// give back the visit of every child on the first `depth` path entries (:291-311)
__device__ __forceinline__ void rollback(const int *path, int depth, int lane, const int *edge_child_id, int *node_inflight,
                                         long long tree_nodes_base, long long tree_edges_base, int node_cnt, int edges) {
    for (int d = lane; d < depth; d += 32) {
        const int enc = path[d];
        if (enc < 0) continue;
        const int parent = enc >> 8, slot = enc & 0xFF;
        if (parent < node_cnt && slot < edges) {
            const int child = edge_child_id[tree_edges_base + (long long)parent * edges + slot];
            if (child >= 0 && child < node_cnt) atomicSub(&node_inflight[tree_nodes_base + child], 1);
        }
    }
}

// PRECLAIM: true = _select_kernel_native, false = the counter-CAS variant
template <bool PRECLAIM>
__global__ void select_kernel(float cpuct, float c_pw, float alpha_pw, const int *__restrict__ edge_child_id,
                              const float *__restrict__ edge_prior, const float *__restrict__ edge_W,
                              const int *__restrict__ edge_N, int *node_inflight, int *node_expand_inflight,
                              const int *__restrict__ node_expanded, const int *__restrict__ tree_nodes, int *out_selected_node,
                              int *out_path_eids, int *out_path_len, int trees, int nodes, int edges, int warps, int path_depth) {
    const int lane = threadIdx.x & 31;
    const int traversal = blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5);
    const int tree = traversal / warps;
    const int wid = traversal - tree * warps;
    if (tree >= trees) return;
    int *path = out_path_eids + (long long)traversal * path_depth;
    int result = PACKED_INVALID, result_len = 0;
    const int node_cnt = tree_nodes[tree];
    const bool shape_ok = path_depth >= 1 && nodes > 0 && node_cnt > 0 && node_cnt <= nodes && node_cnt <= NODE_LIMIT && edges > 0 &&
                          edges <= EDGE_LIMIT;
    const long long tree_nodes_base = (long long)tree * nodes;
    const long long tree_edges_base = tree_nodes_base * edges;
    int node = 0, depth = 0;
    while (shape_ok) {
        if (node < 0 || node >= node_cnt) {
            rollback(path, depth, lane, edge_child_id, node_inflight, tree_nodes_base, tree_edges_base, node_cnt, edges);
            break;
        }
        if (depth >= path_depth) {
            result = pack(DEPTH_LIMIT, node, 0);
            result_len = depth + 1;
            break;
        }
        const int info = node_expanded[tree_nodes_base + node];
        if (info == NODE_TERMINAL) {
            result = pack(TERMINAL, node, 0);
            result_len = depth + 1;
            break;
        }
        if (info < 0 || info > edges) {
            rollback(path, depth, lane, edge_child_id, node_inflight, tree_nodes_base, tree_edges_base, node_cnt, edges);
            break;
        }
        const int n_exp = info;
        const long long e0 = tree_edges_base + (long long)node * edges;
        // ---- the expanded edges of this node, into registers: edge lane + 32 k in slot k
        int child[EPL], cnt[EPL], seen[EPL];
        float prior[EPL], w[EPL];
        int partial = 0;
#pragma unroll
        for (int k = 0; k < EPL; k++) {
            const int e = lane + 32 * k;
            child[k] = -1;
            cnt[k] = 0;
            seen[k] = 0;
            prior[k] = 0.f;
            w[k] = 0.f;
            if (e < n_exp) {
                const int c = edge_child_id[e0 + e];
                if (c >= 0 && c < node_cnt) {
                    child[k] = c;
                    cnt[k] = edge_N[e0 + e];
                    prior[k] = edge_prior[e0 + e];
                    w[k] = edge_W[e0 + e];
                    seen[k] = *(volatile int *)&node_inflight[tree_nodes_base + c];
                    partial += cnt[k] + seen[k];
                }
            }
        }
        const int parent_eff = max(__reduce_add_sync(FULL, partial), 1);   // :418-427
        // progressive widening (:237-262); the preclaim kernel lets a node without children expand exactly one (:646)
        int allowed = 1;
        if (!PRECLAIM || n_exp != 0) {
            const float quota = (alpha_pw == 0.5f) ? c_pw * sqrtf((float)parent_eff) : c_pw * powf((float)parent_eff, alpha_pw);
            allowed = quota >= (float)edges ? edges : max(1, (int)ceilf(quota));
        }
        if (allowed > n_exp) {
            int slot = -1;   // ticket per node: distinct slots for traversals that expand the same node together (:397-414)
            if (lane == 0) {
                const int s = n_exp + atomicAdd(&node_expand_inflight[tree_nodes_base + node], 1);
                if (s < allowed) slot = s;
                else atomicSub(&node_expand_inflight[tree_nodes_base + node], 1);
            }
            slot = __shfl_sync(FULL, slot, 0);
            if (slot >= 0) {
                result = pack(EXPAND, node, slot);
                result_len = depth + 1;
            } else {
                rollback(path, depth, lane, edge_child_id, node_inflight, tree_nodes_base, tree_edges_base, node_cnt, edges);
            }
            break;
        }
        const float sqrt_parent = sqrtf((float)parent_eff);
        int best = NO_EDGE, best_child = -1;
        bool held = false;
        if (PRECLAIM) {
            // every candidate's child is visited first, scored with the count it had before, then the losers leave (:448-483)
            const int rot = wid >= n_exp ? wid % n_exp : wid;   // ties go to the edge closest after the warp's index
            unsigned my_key = 0;
            int my_tie = NO_EDGE, my_child = -1;
#pragma unroll
            for (int k = 0; k < EPL; k++) {
                if (child[k] < 0) continue;
                const int old = atomicAdd(&node_inflight[tree_nodes_base + child[k]], 1);
                const float q = cnt[k] > 0 ? w[k] / (float)cnt[k] : 0.0f;
                const float score = q + cpuct * prior[k] * sqrt_parent / (float)(cnt[k] + old + 1);
                if (score == score) {   // a NaN never wins
                    const unsigned key = ordered(score);
                    int tie = lane + 32 * k - rot;
                    if (tie < 0) tie += n_exp;
                    if (key > my_key || (key == my_key && tie < my_tie)) {
                        my_key = key;
                        my_tie = tie;
                        my_child = child[k];
                    }
                }
            }
            const unsigned top = __reduce_max_sync(FULL, my_key);
            const unsigned tie = __reduce_min_sync(FULL, (top != 0u && my_key == top) ? (unsigned)my_tie : 0xFFFFFFFFu);
            if (top != 0u && tie != 0xFFFFFFFFu) {
                best = (int)tie + rot;
                if (best >= n_exp) best -= n_exp;
                best_child = __shfl_sync(FULL, my_child, __ffs(__ballot_sync(FULL, my_key == top && (unsigned)my_tie == tie)) - 1);
            }
#pragma unroll
            for (int k = 0; k < EPL; k++)
                if (child[k] >= 0 && lane + 32 * k != best) atomicSub(&node_inflight[tree_nodes_base + child[k]], 1);
            held = best != NO_EDGE;
        } else {
            int skip = -1;
            for (int attempt = 0; attempt < MAX_RECALC; attempt++) {
                unsigned my_key = 0;
                int my_e = NO_EDGE, my_child = -1;
#pragma unroll
                for (int k = 0; k < EPL; k++) {
                    const int e = lane + 32 * k;
                    if (child[k] < 0 || e == skip) continue;
                    const float q = cnt[k] > 0 ? w[k] / (float)cnt[k] : 0.0f;
                    const float score = q + cpuct * prior[k] * sqrt_parent / (float)(cnt[k] + seen[k] + 1);
                    if (score == score) {
                        const unsigned key = ordered(score);
                        if (key > my_key || (key == my_key && e < my_e)) {   // lowest edge on ties (:110-119)
                            my_key = key;
                            my_e = e;
                            my_child = child[k];
                        }
                    }
                }
                const unsigned top = __reduce_max_sync(FULL, my_key);
                const unsigned e_min = __reduce_min_sync(FULL, (top != 0u && my_key == top) ? (unsigned)my_e : 0xFFFFFFFFu);
                if (top == 0u || e_min == 0xFFFFFFFFu) {
                    if (skip < 0) break;          // nothing to choose from
                    best = skip;                   // only the edge given back is left: take it after all (:533-536)
                    int mine = -1;
#pragma unroll
                    for (int k = 0; k < EPL; k++)
                        if (k == (skip >> 5)) mine = child[k];
                    best_child = __shfl_sync(FULL, mine, skip & 31);
                } else {
                    best = (int)e_min;
                    best_child = __shfl_sync(FULL, my_child, __ffs(__ballot_sync(FULL, my_key == top && (unsigned)my_e == e_min)) - 1);
                }
                // claim: compare-and-swap old -> old + 1 on the child's counter; `conflict` = somebody was there already
                int claim = 0;   // bit 0: held, bit 1: conflict
                if (lane == 0) {
                    int *counter = &node_inflight[tree_nodes_base + best_child];
                    bool can_claim = true, got = false;
                    int old = 0;
                    for (int t = 0; t < MAX_CLAIM_RETRY && !got; t++) {
                        old = *(volatile int *)counter;
                        if (old < 0 || old >= 0x7FFFFFFF) {
                            can_claim = false;
                            break;
                        }
                        got = atomicCAS(counter, old, old + 1) == old;
                    }
                    if (!got && can_claim) {
                        old = atomicAdd(counter, 1);
                        got = true;
                    }
                    claim = (got ? 1 : 0) | ((got && old > 0) ? 2 : 0);
                }
                claim = __shfl_sync(FULL, claim, 0);
                held = claim & 1;
                if (!held) break;
                if (!(claim & 2) || n_exp <= 1 || attempt + 1 >= MAX_RECALC) break;
                if (lane == 0) atomicSub(&node_inflight[tree_nodes_base + best_child], 1);
                __syncwarp();
                skip = best;
                held = false;
                // the counts may have moved: look at them again
#pragma unroll
                for (int k = 0; k < EPL; k++)
                    if (child[k] >= 0) seen[k] = *(volatile int *)&node_inflight[tree_nodes_base + child[k]];
            }
        }
        if (!held || best_child < 0) {
            if (held && !PRECLAIM && lane == 0 && best_child >= 0) atomicSub(&node_inflight[tree_nodes_base + best_child], 1);
            __syncwarp();
            rollback(path, depth, lane, edge_child_id, node_inflight, tree_nodes_base, tree_edges_base, node_cnt, edges);
            break;
        }
        if (lane == 0) path[depth] = (node << 8) | best;
        __syncwarp();
        node = best_child;
        depth++;
    }
    __syncwarp();
    if (lane == 0) {
        out_selected_node[traversal] = result;
        out_path_len[traversal] = result_len;
    }
}

// _backup_kernel_native (:847-927): per path edge the child's visit is given back, the edge gets N += 1 and W += value;
// an EXPAND result returns its ticket.  With values == NULL only the visits and the ticket are released.
__global__ void backup_kernel(int virtual_loss, const int *__restrict__ edge_child_id, float *edge_W, int *edge_N,
                              int *node_inflight, int *node_expand_inflight, const int *__restrict__ tree_nodes,
                              const int *__restrict__ out_selected_node, const int *__restrict__ out_path_eids,
                              const int *__restrict__ out_path_len, const float *__restrict__ path_edge_values, int trees, int nodes,
                              int edges, int warps, int path_depth) {
    const int lane = threadIdx.x & 31;
    const int traversal = blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5);
    const int tree = traversal / warps;
    if (tree >= trees) return;
    const int node_cnt = tree_nodes[tree];
    if (node_cnt <= 0 || node_cnt > nodes || node_cnt > NODE_LIMIT) return;
    const int raw = out_selected_node[traversal];
    if (raw < 0 || (raw >> KIND_SHIFT) == INVALID) return;
    const int plen = out_path_len[traversal];
    if (plen <= 0) return;
    const long long tree_nodes_base = (long long)tree * nodes, tree_edges_base = tree_nodes_base * edges;
    const int *path = out_path_eids + (long long)traversal * path_depth;
    for (int d = lane; d < plen - 1; d += 32) {
        const int enc = path[d];
        if (enc < 0) continue;
        const int parent = enc >> 8, slot = enc & 0xFF;
        if (parent < node_cnt && slot < edges) {
            const long long ix = tree_edges_base + (long long)parent * edges + slot;
            const int child = edge_child_id[ix];
            if (child >= 0 && child < node_cnt) atomicSub(&node_inflight[tree_nodes_base + child], virtual_loss);
            if (path_edge_values) {
                atomicAdd(&edge_N[ix], 1);
                atomicAdd(&edge_W[ix], path_edge_values[(long long)traversal * path_depth + d]);
            }
        }
    }
    if (lane == 0 && (raw >> KIND_SHIFT) == EXPAND) {
        const int leaf = raw & NODE_MASK;
        if (leaf < node_cnt) atomicSub(&node_expand_inflight[tree_nodes_base + leaf], 1);
    }
}

}  // namespace puct_v2

// variant 0: preclaim (the reference's _select_kernel_native), 1: counter-CAS (_select_kernel_winner_recalc of
// src/puct/puct_gpu_v2.py).  Array shapes as for puct_select_winner_recalc_launch, with node_inflight int32[trees][nodes]
// in place of the per-edge counters.
extern "C" int puct_v2_select_launch(int variant, float cpuct, float c_pw, float alpha_pw, const int *edge_child_id,
                                     const float *edge_prior, const float *edge_W, const int *edge_N, int *node_inflight,
                                     int *node_expand_inflight, const int *node_expanded, const int *tree_nodes,
                                     int *out_selected_node, int *out_path_eids, int *out_path_len, int trees, int nodes, int edges,
                                     int warps, int path_depth, void *stream) {
    if (trees <= 0 || warps <= 0 || warps > 32 || (variant != 0 && variant != 1)) return (int)cudaErrorInvalidValue;
    const unsigned grid = (unsigned)((long long)trees * warps);
    cudaStream_t s = (cudaStream_t)stream;
    if (variant == 0)
        puct_v2::select_kernel<true><<<grid, 32, 0, s>>>(cpuct, c_pw, alpha_pw, edge_child_id, edge_prior, edge_W, edge_N, node_inflight,
                                                         node_expand_inflight, node_expanded, tree_nodes, out_selected_node,
                                                         out_path_eids, out_path_len, trees, nodes, edges, warps, path_depth);
    else
        puct_v2::select_kernel<false><<<grid, 32, 0, s>>>(cpuct, c_pw, alpha_pw, edge_child_id, edge_prior, edge_W, edge_N, node_inflight,
                                                          node_expand_inflight, node_expanded, tree_nodes, out_selected_node,
                                                          out_path_eids, out_path_len, trees, nodes, edges, warps, path_depth);
    return (int)cudaGetLastError();
}

extern "C" int puct_v2_backup_launch(int virtual_loss, const int *edge_child_id, float *edge_W, int *edge_N, int *node_inflight,
                                     int *node_expand_inflight, const int *tree_nodes, const int *out_selected_node,
                                     const int *out_path_eids, const int *out_path_len, const float *path_edge_values, int trees,
                                     int nodes, int edges, int warps, int path_depth, void *stream) {
    if (trees <= 0 || warps <= 0 || warps > 32) return (int)cudaErrorInvalidValue;
    const unsigned grid = (unsigned)((long long)trees * warps);
    puct_v2::backup_kernel<<<grid, 32, 0, (cudaStream_t)stream>>>(virtual_loss, edge_child_id, edge_W, edge_N, node_inflight,
                                                                 node_expand_inflight, tree_nodes, out_selected_node,
                                                                 out_path_eids, out_path_len, path_edge_values, trees, nodes, edges,
                                                                 warps, path_depth);
    return (int)cudaGetLastError();
}
