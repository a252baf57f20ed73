/*
 * puct_b200.h -- C ABI of the warp-level PUCT select in libmctsnc_b200.so (sm_100a).
 *
 * The two first entry points keep name, arguments and meaning of the reference's only native library
 * (src/puct/puct_gpu_v3_cpp.cu), so its ctypes binding (src/puct/puct_gpu_v3_cpp.py:84-156) can load this library in
 * its place.  All pointers are DEVICE pointers; arrays are row-major:
 *   edge_child_id, edge_N, edge_inflight : int32[trees][nodes][edges]     edge_prior, edge_W : float32[trees][nodes][edges]
 *   node_expanded, node_expand_inflight  : int32[trees][nodes]            tree_nodes         : int32[trees]
 *   out_selected_node, out_path_len      : int32[trees][warps]            out_path_eids      : int32[trees][warps][path_depth]
 * Limits: nodes per tree <= 16384, edges <= 256, warps <= 32.  Return value: cudaError_t as int (0 = launched).
 */
#ifndef PUCT_B200_H
#define PUCT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces puct_select_winner_recalc_launch, src/puct/puct_gpu_v3_cpp.cu:450-481 (kernel :277-448; numba twin
   src/puct/puct_gpu_v3.py:426-630): one warp per traversal, grid = trees, block = warps * 32, on `stream`. */
int puct_select_winner_recalc_launch(float cpuct, float c_pw, float alpha_pw, int soft_winner, const int *edge_child_id,
                                     const float *edge_prior, const float *edge_W, const int *edge_N, int *edge_inflight,
                                     int *node_expand_inflight, const int *node_expanded, const int *tree_nodes,
                                     int *out_selected_node, int *out_path_eids, int *out_path_len, int trees, int nodes,
                                     int edges, int warps, int path_depth, void *stream);

/* Replaces puct_cpp_cuda_error_string, src/puct/puct_gpu_v3_cpp.cu:483-485. */
const char *puct_cpp_cuda_error_string(int code);

/* The same select with a virtual-loss weight other than 1.  The reference's select always claims 1
   (src/puct/puct_gpu_v3_cpp.cu:257, :270, :397); only its backup / release kernels take a weight
   (src/puct/puct_gpu_v2.py:854).  An extension, used by the benchmark configuration with virtual loss 3. */
int puct_select_virtual_loss_launch(float cpuct, float c_pw, float alpha_pw, int soft_winner, int virtual_loss,
                                    const int *edge_child_id, const float *edge_prior, const float *edge_W, const int *edge_N,
                                    int *edge_inflight, int *node_expand_inflight, const int *node_expanded,
                                    const int *tree_nodes, int *out_selected_node, int *out_path_eids, int *out_path_len,
                                    int trees, int nodes, int edges, int warps, int path_depth, void *stream);

/* Replaces _backup_kernel_native, src/puct/puct_gpu_v2.py:847-927, for the per-edge inflight layout of v3: per path
   edge inflight -= virtual_loss, N += 1, W += value; an EXPAND result returns its ticket.  path_edge_values:
   float32[trees][warps][path_depth]; NULL releases the claims only (_release_claims_kernel,
   src/puct/test_puct_gpu_v3.py:274-332). */
int puct_backup_launch(int virtual_loss, float *edge_W, int *edge_N, int *edge_inflight, int *node_expand_inflight,
                       const int *tree_nodes, const int *out_selected_node, const int *out_path_eids, const int *out_path_len,
                       const float *path_edge_values, int trees, int nodes, int edges, int warps, int path_depth, void *stream);

/* Replaces the two older select kernels of the reference, for trees that keep virtual visits per child NODE
   (node_inflight: int32[trees][nodes]) instead of per edge:
     variant 0 (preclaim)     _select_kernel_native,        src/puct/puct_gpu_v2.py:573-697
     variant 1 (counter-CAS)  _select_kernel_winner_recalc, src/puct/puct_gpu_v2.py:700-840
   The reference launches them from Python as kernel[trees, warps * 32](cpuct, c_pw, alpha_pw, arrays...) with the shapes
   taken from the arrays (src/puct/test_puct_gpu_v2.py:320-354); here the shapes are arguments, as in the v3 launcher.
   Results: (kind << 22) | (slot << 14) | node with kinds INVALID 0, EXPAND 1, TERMINAL 2, DEPTH_LIMIT 3 (no reason bits,
   no BUSY kind); path entries (parent << 8) | slot; a failed traversal gives back every visit it made. */
int puct_v2_select_launch(int variant, float cpuct, float c_pw, float alpha_pw, const int *edge_child_id, const float *edge_prior,
                          const float *edge_W, const int *edge_N, int *node_inflight, int *node_expand_inflight,
                          const int *node_expanded, const int *tree_nodes, int *out_selected_node, int *out_path_eids,
                          int *out_path_len, int trees, int nodes, int edges, int warps, int path_depth, void *stream);

/* Replaces _backup_kernel_native, src/puct/puct_gpu_v2.py:847-927 (per-node layout): per path edge the child's visits
   -= virtual_loss, N += 1, W += value; an EXPAND result returns its ticket.  path_edge_values == NULL releases only. */
int puct_v2_backup_launch(int virtual_loss, const int *edge_child_id, float *edge_W, int *edge_N, int *node_inflight,
                          int *node_expand_inflight, const int *tree_nodes, const int *out_selected_node, const int *out_path_eids,
                          const int *out_path_len, const float *path_edge_values, int trees, int nodes, int edges, int warps,
                          int path_depth, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PUCT_B200_H */
