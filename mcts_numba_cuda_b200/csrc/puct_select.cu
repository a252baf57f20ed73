// Warp-level PUCT select with virtual loss, plus the backup / release kernels that undo the claims.
//
// Drop-in for the reference's only native library, src/puct/puct_gpu_v3_cpp.cu: the exported launcher
// puct_select_winner_recalc_launch has the same 21 arguments (:450-481) and puct_cpp_cuda_error_string the same
// meaning (:483-485), so the reference's ctypes binding (src/puct/puct_gpu_v3_cpp.py:84-156) can load this library
// instead.  Semantics followed (not the code): one warp = one traversal of its tree; per level the progressive-widening
// quota ceil(c_pw * N^alpha) (:150-157), an expansion ticket by atomicAdd (:219-233), the score
// W/N + cpuct * P * sqrt(N_parent_eff) / (1 + N + inflight) (:171-180), ties broken by edge id rotated by the warp id
// (:50-71), the winner claimed with atomicCAS(inflight, seen, seen + 1) and at most two evaluations (:235-275), the
// path entry (node << 8) | edge (:436), the packed result reason << 25 | kind << 22 | slot << 14 | node (:38-41),
// and the rollback of every claim of the traversal when it fails (:206-217).
//
// What is done differently: the traversal is latency-bound (dependent loads from gigabytes of edge arrays), so a level
// is built to cost ONE memory round trip instead of four.  Every lane keeps child / prior / W / N / inflight of its
// edges in registers; the parent count and the arg-max both come from those registers; and as soon as the winner is
// known, the claim (atomicCAS), the child's node record and ALL the child's edges are requested together, so that the
// next level starts with its data already on the way.  A retry after a lost CAS reloads only `inflight`.  Sums and
// maxima use the warp-reduce instructions (redux.sync) instead of five rounds of three shuffles; the tie-break is a
// second redux over the lanes that hold the maximum.
#include <cuda_runtime.h>
#include <stdint.h>

namespace puct {

constexpr unsigned FULL = 0xFFFFFFFFu;
constexpr int NODE_TERMINAL = -1;
constexpr int NODE_LIMIT = 16384, NODE_MASK = 0x3FFF, EDGE_LIMIT = 256;
constexpr int KIND_SHIFT = 22, SLOT_SHIFT = 14, REASON_SHIFT = 25;
enum Kind { INVALID = 0, EXPAND = 1, TERMINAL = 2, DEPTH_LIMIT = 3, BUSY = 4 };
enum Reason {
    R_UNSET = 0, R_OK_EXPAND = 1, R_OK_TERMINAL = 2, R_OK_DEPTH_LIMIT = 3, R_BUSY_EXPAND_INFLIGHT = 4,
    R_BUSY_WINNER_RECALC = 5, R_INVALID_SHAPE = 10, R_INVALID_NODE_INFO = 11, R_INVALID_NO_VALID_EDGE = 14,
    R_INVALID_CHILD_OOB = 15, R_INVALID_UNKNOWN = 16
};
constexpr int MAX_EVALUATIONS = 2;
#ifndef PUCT_SELECT_WARPS_PER_BLOCK
#define PUCT_SELECT_WARPS_PER_BLOCK 1
#endif
constexpr int SELECT_WARPS_PER_BLOCK = PUCT_SELECT_WARPS_PER_BLOCK;  // traversals per thread block of the select kernel
constexpr float LOWEST = -3.4028234663852886e38f;
constexpr int NO_EDGE = 0x7FFFFFFF;

__device__ __forceinline__ int pack(int kind, int node, int slot, int reason) {
    return (reason << REASON_SHIFT) | (kind << KIND_SHIFT) | (slot << SLOT_SHIFT) | node;
}

__device__ __forceinline__ unsigned ordered(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// undo the claims of the first `depth` path entries of this warp
__device__ __forceinline__ void rollback(const int *path, int depth, int lane, int *edge_inflight, long long tree_edges_base,
                                         int node_cnt, int edges, int amount) {
    for (int d = lane; d < depth; d += 32) {
        const int enc = path[d];
        const int parent = enc >> 8, slot = enc & 0xFF;
        if (parent >= 0 && parent < node_cnt && slot < edges)
            atomicSub(&edge_inflight[tree_edges_base + (long long)parent * edges + slot], amount);
    }
}

// the edges of one node as seen by one lane (edge lane + 32 k in slot k)
template <int EPL>
struct EdgeRegs {
    float prior[EPL], w[EPL];
    int n[EPL], inflight[EPL], child[EPL];
};

// requests all `edges` slots of a node, expanded or not (the arrays are dense, so the addresses are valid): used
// before the node's record has arrived, i.e. before the number of expanded edges is known
template <int EPL>
__device__ __forceinline__ void load_edges(EdgeRegs<EPL> &r, long long e0, int lane, int edges, const int *edge_child_id,
                                           const float *edge_prior, const float *edge_W, const int *edge_N,
                                           const int *edge_inflight) {
#pragma unroll
    for (int k = 0; k < EPL; k++) {
        const int e = lane + 32 * k;
        r.n[k] = 0;
        r.inflight[k] = 0;
        r.prior[k] = 0.f;
        r.w[k] = 0.f;
        r.child[k] = -1;
        if (e < edges) {
            r.child[k] = edge_child_id[e0 + e];
            r.n[k] = edge_N[e0 + e];
            r.inflight[k] = *(volatile const int *)&edge_inflight[e0 + e];
            r.prior[k] = edge_prior[e0 + e];
            r.w[k] = edge_W[e0 + e];
        }
    }
}

// EPL: edges per lane, ceil(edges / 32) rounded up to 1, 2, 4 or 8 (registers follow it)
template <int VL_GENERAL, int EPL>
__global__ void select_kernel(float cpuct, float c_pw, float alpha_pw, int soft_winner, const int *__restrict__ edge_child_id,
                              const float *__restrict__ edge_prior, const float *__restrict__ edge_W,
                              const int *__restrict__ edge_N, int *edge_inflight, int *node_expand_inflight,
                              const int *__restrict__ node_expanded, const int *__restrict__ tree_nodes, int *out_selected_node,
                              int *out_path_eids, int *out_path_len, int trees, int nodes, int edges, int warps,
                              int path_depth, int virtual_loss) {
    // Traversal i = tree * warps + w is run by warp i of the grid, in blocks of SELECT_WARPS_PER_BLOCK warps.  The reference
    // puts the `warps` traversals of a tree into one block (src/puct/puct_gpu_v3_cpp.cu:472-473); with 8 traversals per
    // tree most of them lose the claim at the root and leave after two evaluations, and a block of 8 warps then keeps
    // its 6 idle warp slots until its last traversal has gone all the way down.  Small blocks give the slots back at
    // once; the traversals of a tree still start together (their warps are neighbours in the grid).  Measured on 4096
    // trees x 64 edges x depth 16 with 8 / 1 traversals per tree: one warp per block 0.140 / 0.054 ms, two 0.140 / 0.060,
    // four 0.149 / 0.057, eight (the reference's shape for 8) 0.307 / 0.079; the reference kernel 0.260 / 0.081.
    const int lane = threadIdx.x & 31;
    const int traversal = blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5);
    const int tree = traversal / warps;
    const int wid = traversal - tree * warps;
    const int vl = VL_GENERAL ? virtual_loss : 1;
    if (tree >= trees) return;
    const int out_ix = traversal;
    int *path = out_path_eids + (long long)out_ix * path_depth;
    const int node_cnt = tree_nodes[tree];
    if (!(path_depth >= 1 && nodes > 0 && node_cnt > 0 && node_cnt <= nodes && node_cnt <= NODE_LIMIT && edges > 0 &&
          edges <= EDGE_LIMIT)) {
        if (lane == 0) {
            out_selected_node[out_ix] = pack(INVALID, NODE_MASK, 0, R_INVALID_SHAPE);
            out_path_len[out_ix] = 0;
        }
        return;
    }
    const long long tree_nodes_base = (long long)tree * nodes;
    const long long tree_edges_base = tree_nodes_base * edges;
    int result = pack(INVALID, NODE_MASK, 0, R_INVALID_UNKNOWN);
    int result_len = 0;
    int node = 0, depth = 0;
    int info = node_expanded[tree_nodes_base];
    EdgeRegs<EPL> cur, nxt;
    load_edges<EPL>(cur, tree_edges_base, lane, edges, edge_child_id, edge_prior, edge_W, edge_N, edge_inflight);
    nxt = cur;
    for (;;) {
        if (info == NODE_TERMINAL) {
            result = pack(TERMINAL, node, 0, R_OK_TERMINAL);
            result_len = depth + 1;
            break;
        }
        if (info < 0 || info > edges) {
            rollback(path, depth, lane, edge_inflight, tree_edges_base, node_cnt, edges, vl);
            __syncwarp();
            result = pack(INVALID, NODE_MASK, 0, R_INVALID_NODE_INFO);
            break;
        }
        if (depth >= path_depth) {
            result = pack(DEPTH_LIMIT, node, 0, R_OK_DEPTH_LIMIT);
            result_len = depth + 1;
            break;
        }
        const int n_exp = info;
        const long long e0 = tree_edges_base + (long long)node * edges;
        // ---- the edges of this node are in registers already (requested while the level above was being decided)
        int partial = 0;
        const bool need_stats = n_exp != 1 || c_pw != 0.0f;
#pragma unroll
        for (int k = 0; k < EPL; k++)
            if (lane + 32 * k < n_exp) partial += cur.n[k] + cur.inflight[k];
        int parent_eff = 1, allowed = 1;
        if (need_stats) {
            parent_eff = max(__reduce_add_sync(FULL, partial), 1);
            const float quota = (alpha_pw == 0.5f) ? c_pw * sqrtf((float)parent_eff) : c_pw * powf((float)parent_eff, alpha_pw);
            allowed = quota >= (float)edges ? edges : max(1, (int)ceilf(quota));
        }
        if (allowed > n_exp) {
            // room for a new child: take a ticket unless the tickets in flight already fill the quota
            int slot = -1;
            if (lane == 0) {
                int *tickets = &node_expand_inflight[tree_nodes_base + node];
                if (n_exp + *tickets < allowed) {
                    const int s = n_exp + atomicAdd(tickets, 1);
                    if (s < allowed) slot = s;
                    else atomicSub(tickets, 1);
                }
            }
            slot = __shfl_sync(FULL, slot, 0);
            if (slot >= 0) {
                result = pack(EXPAND, node, slot, R_OK_EXPAND);
                result_len = depth + 1;
                break;
            }
            if (n_exp == 0) {
                rollback(path, depth, lane, edge_inflight, tree_edges_base, node_cnt, edges, vl);
                __syncwarp();
                result = pack(BUSY, node, 0, R_BUSY_EXPAND_INFLIGHT);
                result_len = 0;
                break;
            }
        }
        // ---- pick an existing child
        // The child of every edge is in a register already, so as soon as the winner is known its node record can be
        // requested together with the claim instead of after it: one memory round trip per level less.
        int best = 0, held = 0, child = -1, next_info = 0;
        if (n_exp == 1) {
            child = __shfl_sync(FULL, cur.child[0], 0);
            if (child >= 0 && child < node_cnt) {
                next_info = node_expanded[tree_nodes_base + child];
                load_edges<EPL>(nxt, tree_edges_base + (long long)child * edges, lane, edges, edge_child_id, edge_prior, edge_W,
                                edge_N, edge_inflight);
            }
            if (lane == 0) atomicAdd(&edge_inflight[e0], vl);
            held = 1;
        } else {
            const int rot = wid >= n_exp ? wid % n_exp : wid;  // ties go to the edge closest after `rot`
            const float sqrt_parent = sqrtf((float)parent_eff);
            for (int attempt = 0;; attempt++) {
                unsigned my_key = 0;
                int my_tie = NO_EDGE, my_seen = 0, my_child = -1;
#pragma unroll
                for (int k = 0; k < EPL; k++) {
                    const int e = lane + 32 * k;
                    if (e < n_exp) {
                        const float q = cur.n[k] > 0 ? cur.w[k] / (float)cur.n[k] : 0.0f;
                        const float u = cpuct * cur.prior[k] * sqrt_parent / (float)(cur.n[k] + cur.inflight[k] + 1);
                        const float score = q + u;
                        if (score >= LOWEST) {  // not NaN, not -inf
                            const unsigned key = ordered(score);
                            int tie = e - rot;
                            if (tie < 0) tie += n_exp;
                            if (key > my_key || (key == my_key && tie < my_tie)) {
                                my_key = key;
                                my_tie = tie;
                                my_seen = cur.inflight[k];
                                my_child = cur.child[k];
                            }
                        }
                    }
                }
                const unsigned top = __reduce_max_sync(FULL, my_key);
                const int tie = (int)__reduce_min_sync(FULL, (my_key == top && my_tie != NO_EDGE) ? (unsigned)my_tie : 0xFFFFFFFFu);
                if (top == 0u || tie < 0) {
                    best = NO_EDGE;
                    break;
                }
                best = tie + rot;
                if (best >= n_exp) best -= n_exp;
                const int owner = __ffs(__ballot_sync(FULL, my_key == top && my_tie == tie)) - 1;
                const int seen = __shfl_sync(FULL, my_seen, owner);
                child = __shfl_sync(FULL, my_child, owner);
                if (child >= 0 && child < node_cnt) {  // the next level's data travels together with the claim
                    next_info = node_expanded[tree_nodes_base + child];
                    load_edges<EPL>(nxt, tree_edges_base + (long long)child * edges, lane, edges, edge_child_id, edge_prior,
                                    edge_W, edge_N, edge_inflight);
                }
                if (lane == 0) held = atomicCAS(&edge_inflight[e0 + best], seen, seen + vl) == seen ? 1 : 0;
                held = __shfl_sync(FULL, held, 0);
                if (held || attempt + 1 >= MAX_EVALUATIONS) break;
                // somebody else moved the winner's count: look at the counts again
#pragma unroll
                for (int k = 0; k < EPL; k++) {
                    const int e = lane + 32 * k;
                    if (e < n_exp) cur.inflight[k] = *(volatile int *)&edge_inflight[e0 + e];
                }
            }
            if (soft_winner != 0 && !held && best != NO_EDGE) {
                if (lane == 0) atomicAdd(&edge_inflight[e0 + best], vl);
                held = 1;
            }
        }
        if (!held) {
            __syncwarp();
            rollback(path, depth, lane, edge_inflight, tree_edges_base, node_cnt, edges, vl);
            __syncwarp();
            result = best == NO_EDGE ? pack(INVALID, NODE_MASK, 0, R_INVALID_NO_VALID_EDGE) : pack(BUSY, node, 0, R_BUSY_WINNER_RECALC);
            break;
        }
        if (child < 0 || child >= node_cnt) {
            if (lane == 0) atomicSub(&edge_inflight[e0 + best], vl);
            __syncwarp();
            rollback(path, depth, lane, edge_inflight, tree_edges_base, node_cnt, edges, vl);
            __syncwarp();
            result = pack(INVALID, NODE_MASK, 0, R_INVALID_CHILD_OOB);
            break;
        }
        if (lane == 0) path[depth] = (node << 8) | best;
        __syncwarp();
        node = child;
        info = next_info;
        cur = nxt;
        depth++;
    }
    if (lane == 0) {
        out_selected_node[out_ix] = result;
        out_path_len[out_ix] = result_len;
    }
}

// Turns the claims of finished traversals into statistics (v3 edge layout; the reference has this step only for its
// older node-inflight layout, src/puct/puct_gpu_v2.py:847-927): per path edge inflight -= virtual_loss, N += 1,
// W += value; an EXPAND result also returns its ticket.  With values == NULL only the claims are released
// (src/puct/test_puct_gpu_v3.py:274-332).
__global__ void backup_kernel(int virtual_loss, float *edge_W, int *edge_N, int *edge_inflight, int *node_expand_inflight,
                              const int *__restrict__ tree_nodes, const int *__restrict__ out_selected_node,
                              const int *__restrict__ out_path_eids, const int *__restrict__ out_path_len,
                              const float *__restrict__ path_edge_values, int trees, int nodes, int edges, int warps,
                              int path_depth) {
    const int tree = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int wid = threadIdx.x >> 5;
    if (tree >= trees || wid >= min((int)(blockDim.x >> 5), warps)) return;
    const int node_cnt = tree_nodes[tree];
    if (node_cnt <= 0 || node_cnt > nodes || node_cnt > NODE_LIMIT) return;
    const int out_ix = tree * warps + wid;
    const int raw = out_selected_node[out_ix];
    if (raw < 0) return;
    const int kind = (raw >> KIND_SHIFT) & 7;
    if (kind == INVALID || kind == BUSY) return;
    const int plen = out_path_len[out_ix];
    if (plen <= 0) return;
    const long long tree_edges_base = (long long)tree * nodes * edges;
    const int *path = out_path_eids + (long long)out_ix * path_depth;
    for (int d = lane; d < plen - 1; d += 32) {
        const int enc = path[d];
        if (enc < 0) continue;
        const int parent = enc >> 8, slot = enc & 0xFF;
        if (parent < node_cnt && slot < edges) {
            const long long ix = tree_edges_base + (long long)parent * edges + slot;
            atomicSub(&edge_inflight[ix], virtual_loss);
            if (path_edge_values) {
                atomicAdd(&edge_N[ix], 1);
                atomicAdd(&edge_W[ix], path_edge_values[(long long)out_ix * path_depth + d]);
            }
        }
    }
    if (lane == 0 && kind == EXPAND) {
        const int leaf = raw & NODE_MASK;
        if (leaf < node_cnt) atomicSub(&node_expand_inflight[(long long)tree * nodes + leaf], 1);
    }
}

template <int VL>
static int launch_select(float cpuct, float c_pw, float alpha_pw, int soft_winner, int virtual_loss, const int *edge_child_id,
                         const float *edge_prior, const float *edge_W, const int *edge_N, int *edge_inflight,
                         int *node_expand_inflight, const int *node_expanded, const int *tree_nodes, int *out_selected_node,
                         int *out_path_eids, int *out_path_len, int trees, int nodes, int edges, int warps, int path_depth,
                         cudaStream_t stream) {
    const long long traversals = (long long)trees * warps;
    const unsigned grid = (unsigned)((traversals + SELECT_WARPS_PER_BLOCK - 1) / SELECT_WARPS_PER_BLOCK);
#define PUCT_LAUNCH(E)                                                                                                      \
    select_kernel<VL, E><<<grid, SELECT_WARPS_PER_BLOCK * 32, 0, stream>>>(                                                 \
        cpuct, c_pw, alpha_pw, soft_winner, edge_child_id, edge_prior, edge_W, edge_N, edge_inflight, node_expand_inflight, \
        node_expanded, tree_nodes, out_selected_node, out_path_eids, out_path_len, trees, nodes, edges, warps, path_depth,  \
        virtual_loss)
    if (edges <= 32) PUCT_LAUNCH(1);
    else if (edges <= 64) PUCT_LAUNCH(2);
    else if (edges <= 128) PUCT_LAUNCH(4);
    else PUCT_LAUNCH(8);   // more than 256 edges: the kernel itself reports the invalid shape
#undef PUCT_LAUNCH
    return (int)cudaGetLastError();
}

}  // namespace puct

// Same arguments and meaning as puct_select_winner_recalc_launch of src/puct/puct_gpu_v3_cpp.cu:450-481.
extern "C" int puct_select_winner_recalc_launch(float cpuct, float c_pw, float alpha_pw, int soft_winner, const int *edge_child_id,
                                                const float *edge_prior, const float *edge_W, const int *edge_N,
                                                int *edge_inflight, int *node_expand_inflight, const int *node_expanded,
                                                const int *tree_nodes, int *out_selected_node, int *out_path_eids,
                                                int *out_path_len, int trees, int nodes, int edges, int warps, int path_depth,
                                                void *stream) {
    if (trees <= 0 || warps <= 0 || warps > 32) return (int)cudaErrorInvalidValue;
    return puct::launch_select<0>(cpuct, c_pw, alpha_pw, soft_winner, 1, edge_child_id, edge_prior, edge_W, edge_N, edge_inflight,
                                  node_expand_inflight, node_expanded, tree_nodes, out_selected_node, out_path_eids,
                                  out_path_len, trees, nodes, edges, warps, path_depth, (cudaStream_t)stream);
}

// The same select with a virtual-loss weight other than 1 (an extension: the reference's select always claims 1).
extern "C" int puct_select_virtual_loss_launch(float cpuct, float c_pw, float alpha_pw, int soft_winner, int virtual_loss,
                                               const int *edge_child_id, const float *edge_prior, const float *edge_W,
                                               const int *edge_N, int *edge_inflight, int *node_expand_inflight,
                                               const int *node_expanded, const int *tree_nodes, int *out_selected_node,
                                               int *out_path_eids, int *out_path_len, int trees, int nodes, int edges, int warps,
                                               int path_depth, void *stream) {
    if (trees <= 0 || warps <= 0 || warps > 32 || virtual_loss < 1) return (int)cudaErrorInvalidValue;
    return puct::launch_select<1>(cpuct, c_pw, alpha_pw, soft_winner, virtual_loss, edge_child_id, edge_prior, edge_W, edge_N,
                                  edge_inflight, node_expand_inflight, node_expanded, tree_nodes, out_selected_node,
                                  out_path_eids, out_path_len, trees, nodes, edges, warps, path_depth, (cudaStream_t)stream);
}

// Backup of finished traversals (path_edge_values: float[trees][warps][path_depth], already seen from the side of the
// player who took the edge) or, with path_edge_values == NULL, release of their claims only.
extern "C" int puct_backup_launch(int virtual_loss, float *edge_W, int *edge_N, int *edge_inflight, int *node_expand_inflight,
                                  const int *tree_nodes, const int *out_selected_node, const int *out_path_eids,
                                  const int *out_path_len, const float *path_edge_values, int trees, int nodes, int edges,
                                  int warps, int path_depth, void *stream) {
    if (trees <= 0 || warps <= 0 || warps > 32) return (int)cudaErrorInvalidValue;
    puct::backup_kernel<<<trees, warps * 32, 0, (cudaStream_t)stream>>>(virtual_loss, edge_W, edge_N, edge_inflight,
                                                                       node_expand_inflight, tree_nodes, out_selected_node,
                                                                       out_path_eids, out_path_len, path_edge_values, trees,
                                                                       nodes, edges, warps, path_depth);
    return (int)cudaGetLastError();
}

// Same meaning as puct_cpp_cuda_error_string of src/puct/puct_gpu_v3_cpp.cu:483-485.
extern "C" const char *puct_cpp_cuda_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }
