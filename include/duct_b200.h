/*
 * duct_b200.h -- C ABI of the decoupled-UCT (DUCT) select for simultaneous-move games in libmctsnc_b200.so (sm_100a).
 *
 * NO COUNTERPART IN THE REFERENCE.  The reference's src/puct holds a single-agent PUCT select only; nothing in it
 * selects joint actions.  The entry points below implement this library's own specification of the benchmark
 * configuration "DUCT, 2 players x 8 actions"; oracle/duct_oracle.py restates it on the CPU.  Conventions shared with
 * puct_b200.h: device pointers, row-major arrays, one warp per traversal, grid = trees, block = warps * 32, path
 * entries (node << 8) | slot, packed results reason << 25 | kind << 22 | slot << 14 | node with
 * kind 1 = expand, 2 = terminal, 3 = depth limit, 4 = busy, 0 = invalid.
 *
 * Arrays (A = actions per player <= 16, joint action of (a0, a1) = a0 * A + a1):
 *   child         : int32[trees][nodes][A * A]    child node of a joint action, -1 = none, -2 = being expanded
 *   node_prior, node_w : float32[trees][nodes][2][A]   per player and action: prior, sum of values (own point of view)
 *   node_n, node_inflight : int32[trees][nodes][2][A]  visit count, traversals in flight
 *   node_terminal : int32[trees][nodes]           tree_nodes : int32[trees]
 *   out_selected, out_len : int32[trees][warps]   out_path : int32[trees][warps][path_depth]
 *
 * Select, per level: for each player p and action a
 *     n' = n + vl * inflight,  w' = w - vl * inflight,  q = n' > 0 ? w' / n' : 0,
 *     score = q + (cpuct * prior * sqrt(max(sum_a n', 1))) / (1 + n')        (float32, every operation rounded once)
 * each player takes its arg-max (lowest action on ties), both claims are added to node_inflight (+vl), the path entry
 * is written, and the traversal follows child[joint].  A claim is a compare-and-swap on the in-flight count the action
 * was scored with; when another traversal got there first the player's counts are read again and its arg-max is redone
 * (the third evaluation claims unconditionally), so concurrent traversals spread like consecutive ones.  A traversal
 * that is alone in its tree never retries.  It ends at a terminal node (kind 2), at path_depth entries
 * (kind 3), or at a joint action without child: the traversal that flips the slot from -1 to -2 returns kind 1 with
 * (node, joint); any other returns kind 4 after giving back all its claims (path length 0).
 *
 * Backup, per path entry: node_inflight -= vl for both players' actions; if `values` is given (float32[trees][warps]
 * [path_depth], from player 0's point of view) node_n += 1 for both, node_w += v for player 0 and -v for player 1.
 * A kind-1 result gets new_child[tree][warp] installed in its slot when that is given and >= 0, else the slot returns
 * to -1.  Return value: cudaError_t as int (0 = launched).
 */
#ifndef DUCT_B200_H
#define DUCT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

int duct_select_launch(float cpuct, int virtual_loss, int *child, const float *node_prior, const float *node_w,
                       const int *node_n, int *node_inflight, const int *node_terminal, const int *tree_nodes,
                       int *out_selected, int *out_path, int *out_len, int trees, int nodes, int actions, int warps,
                       int path_depth, void *stream);

int duct_backup_launch(int virtual_loss, int *child, float *node_w, int *node_n, int *node_inflight, const int *out_selected,
                       const int *out_path, const int *out_len, const float *values, const int *new_child, int trees, int nodes,
                       int actions, int warps, int path_depth, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DUCT_B200_H */
