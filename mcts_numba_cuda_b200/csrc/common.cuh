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
};

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
};

}  // namespace mctsnc
