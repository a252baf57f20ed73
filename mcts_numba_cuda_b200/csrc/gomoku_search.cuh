// Gomoku (15x15, exactly five in a row wins) search kernels.
//
// A Gomoku tree-step plays out up to 225 children x P games of about 110 plies each: far more than one block can do
// in reasonable time, so a step is two launches that the host enqueues without waiting:
//   tree_step_kernel   one block per tree: backup of the previous step, then select and expand
//                      (_backup_* :2084-2220, _select :1293-1365, _expand_1_* :1368-1681, _expand_2_* :1691-1821)
//   playout_dynamic_kernel  a persistent grid whose lanes take the step's games one by one (_playout_ocp /
//                      _playout_acp_* :1824-2081 with the Gomoku device functions of src/mctsnc_game_mechanics.py:181-281)
// and a last tree_step_kernel launch in backup-only mode.  (Line numbers: src/mctsnc.py of the reference.)
//
// Positions are bitboards: cell (i, j) is bit i*15+j of an 8-word set per player; a node stores 16 words
// (player -1, then player +1).  As for Connect 4 the children of a node occupy consecutive slots in ascending action
// order, so a node stores its first child and the number of children; the child of action a is
// first_child + (number of empty cells below a).
#pragma once
#include "common.cuh"
#include "rng.cuh"

namespace mctsnc {
namespace gomoku {

constexpr int M = 15, N = 15, A = 225;
constexpr int WORDS = 8;  // 32-bit words of one player's stone set

// meta of a Gomoku node: bits 0..7 number of children (0 = leaf), bit 8 terminal, bits 9..10 outcome + 1, bit 11 turn,
// bits 16..31 depth
constexpr int G_NCHILD_MASK = 0xFF;
constexpr int G_TERMINAL = 1 << 8;
constexpr int G_OUTCOME_SHIFT = 9;
constexpr int G_TURN_POS = 1 << 11;
__host__ __device__ __forceinline__ int g_outcome(int meta) { return ((meta >> G_OUTCOME_SHIFT) & 3) - 1; }
__host__ __device__ __forceinline__ int g_turn(int meta) { return (meta & G_TURN_POS) ? 1 : -1; }
__host__ __device__ __forceinline__ int g_make_meta(int n_children, bool terminal, int outcome, int turn, int depth) {
    return n_children | (terminal ? G_TERMINAL : 0) | ((outcome + 1) << G_OUTCOME_SHIFT) | (turn > 0 ? G_TURN_POS : 0) |
           (depth << META_DEPTH_SHIFT);
}

// what one step leaves for the playout kernel and for the backup that follows it
struct StepInfo {
    int selected;
    int mode;         // MODE_ALL_CHILDREN / MODE_TERMINAL / MODE_TREE_FULL
    int n_exp;
    int first_child;
    int sel_meta;
    int path_len;
    int pick;         // OCP: rank of the child that is played out
    int pending;      // 1: playouts of this step have been launched, their backup is still to be done
    int n_active;     // children that need real playouts this step (their ranks: Params::active_rank)
    int game_counter; // next game of the step to hand out (game = active child index * P + t)
    int n_empty;      // empty cells of the selected node's position
};

struct Params {
    int4 *rec;
    unsigned *board;          // [trees][cap][16]
    int *parent;
    TreeState *state;
    StepInfo *step;           // [trees]
    int *paths;               // [trees][PATH_CAP]
    int *path_ns;             // [trees][PATH_CAP]
    int *path_wins;           // [trees][PATH_CAP]
    short *actions_expanded;  // [trees][A + 2]
    int *child_out;           // [trees][A][2]   trees_playout_outcomes_children / per-child tallies of the step
    signed char *child_outcome;  // [trees][A]   by rank: outcome of the child (2 = ongoing)
    unsigned char *child_action; // [trees][A]   by rank: action of the child
    unsigned char *active_rank;  // [trees][A]   ranks of the children that need real playouts, ascending
    unsigned *tpl;               // [trees][TPL_WORDS]  the selected node's position in the form the playouts use
    ulonglong2 *rng_playout;
    ulonglong2 *rng_expand;
    const unsigned *root_board;  // [batch][16]
    const signed char *root_turn;
    long long cap;
    long long node_limit;
    int n_trees;
    int n_playouts;
    int variant;
    int tree_base;            // a launch works on the trees [tree_base, tree_base + its number of trees)
    int first;                // 1: reset the trees to the roots before anything else
    int backup_only;          // 1: only the backup of the pending step
    float ucb_c;
    float ms_per_cycle;       // 1 / (nominal SM clock in kHz), for the stage times of TreeState
};

__device__ __forceinline__ unsigned bitrev8(unsigned x) { return __brev(x) >> 24; }

__device__ __forceinline__ unsigned ordered_key(float v) {
    unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// compute_outcome_gomoku (src/mctsnc_game_mechanics.py:220-272) for one direction, on a line word of the form the playouts
// keep (see below): does the stone that `hs` (0: player -1, 16: player +1) puts at position `pos` make a line of exactly
// five?  The reference counts at most 5 stones either way and wants a total of 4, i.e. a run of exactly five that holds
// the stone; cells that do not exist are never set, so the ends of the board count as empty.
__device__ __forceinline__ bool five_on_line(unsigned word, int hs, int pos) {
    const unsigned u = ((word >> hs) & 0x7FFFu) | (1u << pos);
    const unsigned f = u & (u >> 1) & (u >> 2) & (u >> 3) & (u >> 4);   // bit s: stones at s .. s + 4
    const unsigned e = f & ~(u << 1) & ~(u >> 5);                        // and none at s - 1 and s + 5
    return (e & ((0x1Fu << pos) >> 4)) != 0u;                            // runs that hold pos: s = pos - 4 .. pos
}

// block-wide max of a 32-bit key followed by min of a tie-break value among the threads that hold the max
// (256 threads); returns the winning thread's tie value to every thread
__device__ __forceinline__ unsigned block_argmax(unsigned key, unsigned tie, unsigned *s_red, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    unsigned m = __reduce_max_sync(0xFFFFFFFFu, key);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    unsigned best = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) best = max(best, s_red[w]);
    __syncthreads();
    unsigned t = __reduce_min_sync(0xFFFFFFFFu, key == best ? tie : 0xFFFFFFFFu);
    if (lane == 0) s_red[warp] = t;
    __syncthreads();
    unsigned tbest = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) tbest = min(tbest, s_red[w]);
    __syncthreads();
    return tbest;
}

// ---------------------------------------------------------------------------------------------------------------
// A game in progress, as the playouts keep it (per thread in shared memory; the same words per tree in Params::tpl for
// the selected node, written by the tree step and copied by the playouts):
//   LIST_WORDS words   the list of legal actions, one byte each, in the order the reference's swap-remove leaves them
//                      (src/mctsnc_game_mechanics.py:209-217); the byte of cell (i, j) is i * 16 + j, row and column ready
//                      to use;
//   LINE_WORDS words   the stones by line, one word per line of each of the four directions, stones of -1 in bits 0..14,
//                      stones of +1 in bits 16..30, at the bit of their position along the line:
//                        row i                     (position j)
//                        column j                  (position i)
//                        diagonal (i - j + 14) & 15   (position j)
//                        anti-diagonal (i + j) & 15   (position j)
//                      A stone is set in four words, and the exactly-five test of a direction reads one word.  Cells that do
//                      not exist are never set, so no line needs a mask.  The 29 diagonals fold into 16 words: i - j + 14 =
//                      d <= 12 and d + 16 share a word, d occupies the positions 14 - d .. 14 and d + 16 the positions
//                      0 .. 12 - d, with position 13 - d between them always empty: a run of stones cannot pass from one to
//                      the other and finds the empty position where the board ends.  Likewise i + j = a <= 12 (positions
//                      0 .. a) and a + 16 (positions a + 2 .. 14).
constexpr int LIST_WORDS = 57, LINE_WORDS = 15 + 15 + 16 + 16, THREAD_WORDS = LIST_WORDS + LINE_WORDS;
constexpr int LINE_ROW = LIST_WORDS, LINE_COL = LINE_ROW + 15, LINE_DIAG = LINE_COL + 15, LINE_ANTI = LINE_DIAG + 16;
// Params::tpl keeps the two parts on 16-byte boundaries, so that a playout thread copies them four words at a time
constexpr int TPL_LIST = 0, TPL_LINES = 60, TPL_WORDS = 124;
// Table of the exactly-five test: one byte per 11-cell window of a line (the new stone at bit 5, five cells either way; bit
// k = the mover's stone k - 5 positions along): 1 iff the stones next to the middle add up to exactly 4, which is what the
// reference asks for (it counts at most 5 stones either way and wants a total of 4, src/mctsnc_game_mechanics.py:220-272).
constexpr int FIVE_BYTES = 2048;

// ---------------------------------------------------------------------------------------------------------------
// one block of 256 threads per tree
template <bool OCP>
__global__ void __launch_bounds__(256) tree_step_kernel(const Params p) {
    __shared__ unsigned s_board[16];
    __shared__ unsigned s_lines[15 + 15 + 16 + 16];   // the selected node's stones by line (LINE_WORDS words, see below)
    __shared__ int s_prefix[9];      // empty cells before word w
    __shared__ unsigned s_red[8];
    __shared__ int s_red_i[2][8];
    __shared__ int4 s_rec;
    __shared__ int s_node;
    __shared__ int s_pick;
    const int g = p.tree_base + (int)blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int P = p.n_playouts;
    int4 *rec = p.rec + (long long)g * p.cap;
    unsigned *board = p.board + (long long)g * p.cap * 16;
    int *parent = p.parent + (long long)g * p.cap;
    TreeState *st = p.state + g;
    StepInfo *si = p.step + g;
    int *path = p.paths + g * PATH_CAP;
    int *path_ns = p.path_ns + g * PATH_CAP;
    int *path_wins = p.path_wins + g * PATH_CAP;
    short *ae = p.actions_expanded + g * (A + 2);
    int *child_out = p.child_out + g * A * 2;
    signed char *child_outcome = p.child_outcome + g * A;
    unsigned char *child_action = p.child_action + g * A;
    const bool thrifty = (p.variant == 0 || p.variant == 2);

    if (p.first) {
        const int b = g / p.n_trees;
        if (tid < 16) board[tid] = p.root_board[b * 16 + tid];
        if (tid == 0) {
            const int turn = p.root_turn[b];
            rec[0] = make_int4(0, 0, -1, g_make_meta(0, false, 2, turn, 0));
            parent[0] = -1;
            st->size = 1;
            st->selected = 0;
            st->path_len = 1;
            st->status = 0;
            st->plies = 0;
            st->ub_draws = 0;
            for (int k = 0; k < 4; k++) st->stage_ms[k] = 0.f;
            si->pending = 0;
        }
        __syncthreads();
    }
    const int root_turn = g_turn(rec[0].w);
    const unsigned c_begin = (unsigned)clock();   // stage times: cycle counts of thread 0 (differences modulo 2^32)

    // =============================================================== backup of the step whose playouts have finished
    if (si->pending) {
        const int mode = si->mode, n_exp = si->n_exp, sel_meta = si->sel_meta, first_child = si->first_child;
        const int child_turn = -g_turn(sel_meta);
        const int pick = si->pick;
        int my_neg = 0, my_pos = 0;
        long long n_tot = P;
        if (mode == MODE_ALL_CHILDREN) {
            if (tid < n_exp) {
                const int a = child_action[tid];
                const int o = child_outcome[tid];
                const bool played = !OCP || tid == pick;
                if (played) {
                    if (o == 2) {
                        my_neg = child_out[a * 2 + 0];
                        my_pos = child_out[a * 2 + 1];
                    } else {  // terminal child: its stored outcome stands for all P playouts (:2016-2021)
                        my_neg = o == -1 ? P : 0;
                        my_pos = o == 1 ? P : 0;
                        if (!OCP) {
                            child_out[a * 2 + 0] = my_neg;
                            child_out[a * 2 + 1] = my_pos;
                        }
                    }
                }
                const int cns = played ? P : 0;
                const int cw = played ? (child_turn == 1 ? my_neg : my_pos) : 0;
                rec[first_child + tid] =
                    make_int4(cns, cw, -1, g_make_meta(0, o != 2, o, child_turn, meta_depth(sel_meta) + 1));
            }
            if (!OCP) n_tot = (long long)P * n_exp;
        } else if (mode == MODE_TERMINAL) {
            if (tid == 0) {
                my_neg = st->out_neg;
                my_pos = st->out_pos;
            }
        } else {  // the selected node itself was played out (slot of action 0)
            if (tid == 0) {
                my_neg = child_out[0];
                my_pos = child_out[1];
            }
        }
        int wn = __reduce_add_sync(0xFFFFFFFFu, my_neg), wp = __reduce_add_sync(0xFFFFFFFFu, my_pos);
        if (lane == 0) {
            s_red_i[0][warp] = wn;
            s_red_i[1][warp] = wp;
        }
        __syncthreads();
        int neg_tot = 0, pos_tot = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            neg_tot += s_red_i[0][w];
            pos_tot += s_red_i[1][w];
        }
        const int plen = si->path_len;
        for (int e = tid; e < plen; e += 256) {
            const int node = path[e];
            const int turn_e = (e & 1) ? -root_turn : root_turn;
            const int ns = path_ns[e] + (int)n_tot;
            const int wins = path_wins[e] + (turn_e == 1 ? neg_tot : pos_tot);
            if (e == plen - 1 && mode == MODE_ALL_CHILDREN) rec[node] = make_int4(ns, wins, first_child, sel_meta | n_exp);
            else *reinterpret_cast<int2 *>(&rec[node]) = make_int2(ns, wins);
        }
        __syncthreads();
        if (tid == 0) {
            st->out_neg = neg_tot;
            st->out_pos = pos_tot;
            si->pending = 0;
        }
        __threadfence_block();
        __syncthreads();
    }
    const unsigned c_select = (unsigned)clock();
    if (tid == 0) st->stage_ms[3] += (float)(c_select - c_begin) * p.ms_per_cycle;
    if (p.backup_only) return;

    // =============================================================== select
    if (tid == 0) {
        s_rec = rec[0];
        s_node = 0;
        path[0] = 0;
        path_ns[0] = s_rec.x;
        path_wins[0] = s_rec.y;
    }
    __syncthreads();
    int depth = 0;
    const double c_ucb = (double)p.ucb_c;
    while ((s_rec.w & G_NCHILD_MASK) != 0 && depth < PATH_CAP - 2) {
        const int4 r = s_rec;
        const int node = s_node;
        const int n_children = r.w & G_NCHILD_MASK;
        if (tid < 16) s_board[tid] = board[(long long)node * 16 + tid];
        __syncthreads();
        if (tid == 0) {
            int acc = 0;
            for (int w = 0; w < WORDS; w++) {
                s_prefix[w] = acc;
                const unsigned valid = w == 7 ? 0x1u : 0xFFFFFFFFu;  // 225 = 7*32 + 1
                acc += __popc(~(s_board[w] | s_board[8 + w]) & valid);
            }
            s_prefix[8] = acc;
        }
        __syncthreads();
        unsigned key = 0;
        int child = -1;
        int4 cr = make_int4(0, 0, -1, 0);
        if (tid < A) {
            const int w = tid >> 5, bit = tid & 31;
            const unsigned empty = ~(s_board[w] | s_board[8 + w]);
            if ((empty >> bit) & 1u) {
                const int rank = s_prefix[w] + __popc(empty & ((1u << bit) - 1u));
                if (rank < n_children) {
                    child = r.z + rank;
                    cr = rec[child];
                    float v;
                    if (cr.x == 0) {
                        v = __int_as_float(0x7f800000);
                    } else {
                        // src/mctsnc.py:1337: float64 arithmetic, fused multiply-add, one rounding to float32
                        const double q = (double)cr.y / (double)__int2float_rn(cr.x);
                        const double e = sqrt(log((double)r.x) / (double)cr.x);
                        v = __double2float_rn(fma(c_ucb, e, q));
                    }
                    key = ordered_key(v);
                }
            }
        }
        // ties: the reference's stride-halving reduction keeps the left operand (:1343-1351): smallest bit-reversed index
        const unsigned win_rev = block_argmax(child >= 0 ? key : 0u, child >= 0 ? bitrev8(tid) : 0xFFFFFFFFu, s_red, tid);
        const int winner = (int)bitrev8(win_rev);
        __syncthreads();
        if (tid == winner) {
            s_rec = cr;
            s_node = child;
            path[depth + 1] = child;
            path_ns[depth + 1] = cr.x;
            path_wins[depth + 1] = cr.y;
        }
        depth++;
        __syncthreads();
    }

    // =============================================================== expand
    const unsigned c_expand = (unsigned)clock();
    const int4 r = s_rec;
    const int node = s_node;
    const int sel_turn = g_turn(r.w);
    int mode, n_exp = 0, first_child = -1;
    if (r.w & G_TERMINAL) {
        mode = MODE_TERMINAL;
        if (tid == 0) {
            const int o = g_outcome(r.w);
            st->out_neg = o == -1 ? P : 0;
            st->out_pos = o == 1 ? P : 0;
        }
    } else {
        if (tid < 16) s_board[tid] = board[(long long)node * 16 + tid];
        __syncthreads();
        if (tid == 0) {
            int acc = 0;
            for (int w = 0; w < WORDS; w++) {
                s_prefix[w] = acc;
                const unsigned valid = w == 7 ? 0x1u : 0xFFFFFFFFu;
                acc += __popc(~(s_board[w] | s_board[8 + w]) & valid);
            }
            s_prefix[8] = acc;
        }
        __syncthreads();
        const int n_legal = s_prefix[8];
        {
            // the position in the playouts' form: the list of empty cells in ascending order, the stones by line
            unsigned *tpl = p.tpl + (long long)g * TPL_WORDS;
            unsigned char *tpl_list = reinterpret_cast<unsigned char *>(tpl + TPL_LIST);
            if (tid < A) {
                const int w = tid >> 5, bit = tid & 31;
                const unsigned empty = ~(s_board[w] | s_board[8 + w]);
                if ((empty >> bit) & 1u)
                    tpl_list[s_prefix[w] + __popc(empty & ((1u << bit) - 1u))] = (unsigned char)(((tid / N) << 4) | (tid % N));
            }
            // the line words: one (line, position) pair per thread and round, the cell's stones OR-ed into the line's word
            if (tid < LINE_WORDS) s_lines[tid] = 0u;
            __syncthreads();
            for (int pair = tid; pair < LINE_WORDS * 15; pair += 256) {
                const int lt = pair / 15, pos = pair - lt * 15;
                const int family = lt < 15 ? 0 : (lt < 30 ? 1 : (lt < 46 ? 2 : 3));
                const int idx = lt - (family == 0 ? 0 : (family == 1 ? 15 : (family == 2 ? 30 : 46)));
                unsigned bits = 0;
                for (int fold = 0; fold < 2; fold++) {   // the two lines of a folded word; rows and columns have one
                    int i, j;
                    if (family == 0) {
                        i = idx;
                        j = pos;
                    } else if (family == 1) {
                        i = pos;
                        j = idx;
                    } else if (family == 2) {
                        j = pos;
                        i = idx + 16 * fold - 14 + j;
                    } else {
                        j = pos;
                        i = idx + 16 * fold - j;
                    }
                    if ((family < 2 && fold == 1) || i < 0 || i >= M) continue;
                    const int c = i * N + j;
                    if ((s_board[c >> 5] >> (c & 31)) & 1u) bits |= 1u << pos;
                    if ((s_board[8 + (c >> 5)] >> (c & 31)) & 1u) bits |= 1u << (16 + pos);
                }
                if (bits) atomicOr(&s_lines[lt], bits);
            }
            __syncthreads();
            if (tid < LINE_WORDS) tpl[TPL_LINES + tid] = s_lines[tid];
        }
        const int size = st->size;
        long long room = p.node_limit - (long long)size;
        if (room < 0) room = 0;
        n_exp = n_legal < room ? n_legal : (int)room;
        if (n_exp < n_legal && tid == 0) st->status |= STATUS_TREE_FULL;
        if (n_exp > 0) {
            mode = MODE_ALL_CHILDREN;
            first_child = size;
            if (OCP) {
                if (tid == 0) {
                    // src/mctsnc.py:1435 / :1511: float32 * int64 is a float64 product, truncated
                    ulonglong2 es = p.rng_expand[g];
                    const float u = rng_uniform_f32(es.x, es.y);
                    p.rng_expand[g] = es;
                    int pick = __double2int_rz((double)u * (double)n_exp);
                    if (pick >= n_exp) {  // u == 1.0f: undefined in the reference, clamped
                        pick = n_exp - 1;
                        st->ub_draws += 1;
                        st->status |= STATUS_UB_DRAW;
                    }
                    s_pick = pick;
                }
                __syncthreads();
            }
            bool plays = false;   // this thread's child needs real playouts
            int my_rank = 0;
            if (tid < A) {
                const int w = tid >> 5, bit = tid & 31;
                const unsigned empty = ~(s_board[w] | s_board[8 + w]);
                const bool legal = (empty >> bit) & 1u;
                const int rank = s_prefix[w] + __popc(empty & ((1u << bit) - 1u));
                if (legal && rank < n_exp) {
                    // _expand_2_*: the child's position and outcome (:1794-1821)
                    const int off = sel_turn > 0 ? 8 : 0, hs = sel_turn > 0 ? 16 : 0;
                    const int i = tid / N, j = tid - i * N;
                    const bool win = five_on_line(s_lines[i], hs, j) || five_on_line(s_lines[15 + j], hs, i) ||
                                     five_on_line(s_lines[30 + ((i - j + 14) & 15)], hs, j) ||
                                     five_on_line(s_lines[46 + ((i + j) & 15)], hs, j);
                    const int outcome = win ? sel_turn : (n_legal == 1 ? 0 : 2);
                    uint4 *cb = reinterpret_cast<uint4 *>(board + (long long)(first_child + rank) * 16);
#pragma unroll
                    for (int q = 0; q < 4; q++) {   // the parent's 16 words, the new stone in word off + w
                        uint4 v = make_uint4(s_board[4 * q], s_board[4 * q + 1], s_board[4 * q + 2], s_board[4 * q + 3]);
                        if (((off + w) >> 2) == q) {
                            const unsigned stone = 1u << bit;
                            const int k = (off + w) & 3;
                            v.x |= k == 0 ? stone : 0u;
                            v.y |= k == 1 ? stone : 0u;
                            v.z |= k == 2 ? stone : 0u;
                            v.w |= k == 3 ? stone : 0u;
                        }
                        cb[q] = v;
                    }
                    parent[first_child + rank] = node;
                    child_action[rank] = (unsigned char)tid;
                    child_outcome[rank] = (signed char)outcome;
                    if (!OCP || rank == s_pick) {  // the tallies the playout block adds to
                        child_out[tid * 2 + 0] = 0;
                        child_out[tid * 2 + 1] = 0;
                    }
                    if (thrifty) ae[rank] = (short)tid;
                    else ae[tid] = (short)tid;
                    plays = outcome == 2 && (!OCP || rank == s_pick);
                    my_rank = rank;
                } else if (!thrifty) {
                    ae[tid] = -1;
                }
            }
            // the ranks of the children that are played out, ascending: position = playing children of lower rank
            const unsigned playing_lanes = __ballot_sync(0xFFFFFFFFu, plays);
            if (lane == 0) s_red[warp] = (unsigned)__popc(playing_lanes);
            __syncthreads();
            if (plays) {
                int before = __popc(playing_lanes & ((1u << lane) - 1u));
                for (int wb = 0; wb < warp; wb++) before += (int)s_red[wb];
                p.active_rank[g * A + before] = (unsigned char)my_rank;
            }
        } else {
            mode = MODE_TREE_FULL;
            if (tid == 0) {
                child_out[0] = 0;
                child_out[1] = 0;
            }
            if (tid < A && !thrifty) ae[tid] = -1;
        }
    }
    if (mode == MODE_TERMINAL && tid < A && !thrifty) ae[tid] = -1;
    __syncthreads();
    if (tid == 0) {
        if (mode == MODE_ALL_CHILDREN) st->size += n_exp;
        ae[A + 1] = (short)(mode == MODE_ALL_CHILDREN ? n_exp : 1);
        int m2 = mode;
        const int pick = (OCP && mode == MODE_ALL_CHILDREN) ? s_pick : 0;
        if (OCP && mode == MODE_ALL_CHILDREN) m2 = thrifty ? pick : child_action[pick];
        ae[A] = (short)m2;
        if (!OCP && mode != MODE_ALL_CHILDREN) ae[0] = 0;
        si->selected = node;
        si->mode = mode;
        si->n_exp = n_exp;
        si->first_child = first_child;
        si->sel_meta = r.w;
        si->path_len = depth + 1;
        si->pick = pick;
        int n_active = 0;
        if (mode == MODE_ALL_CHILDREN) {
            for (int wb = 0; wb < 8; wb++) n_active += (int)s_red[wb];
        } else if (mode == MODE_TREE_FULL) {
            p.active_rank[g * A] = 0;
            n_active = 1;
        }
        si->n_active = n_active;
        si->n_empty = mode == MODE_TERMINAL ? 0 : s_prefix[8];
        si->game_counter = 0;
        si->pending = 1;
        st->selected = node;
        st->path_len = depth + 1;
        st->stage_ms[0] += (float)(c_expand - c_select) * p.ms_per_cycle;
        st->stage_ms[1] += (float)((unsigned)clock() - c_expand) * p.ms_per_cycle;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Byte-for-byte emulation of one Gomoku playout of the reference on int8 / int16 local arrays (see the Connect-4
// counterpart): entered only after a uniform draw equal to 1.0f, which makes the reference read the slot one past its
// list of legal actions.  The per-thread list starts as zeros, negative indices wrap once (numba), and the loop gives
// up after 4096 plies (list and board can get out of step for good; the reference would then never return).
struct EmuResult {
    int outcome;
    unsigned plies, ub, err;
    unsigned long long s0, s1;
};

__device__ __forceinline__ int emu_wrap(int i, int len, unsigned &err) {
    if (i < 0) i += len;
    if (i < 0 || i >= len) {
        err = 1;
        i = i < 0 ? 0 : len - 1;
    }
    return i;
}

__device__ __noinline__ EmuResult playout_emulated(const unsigned *start /* 16 words */, int turn, unsigned long long s0,
                                                   unsigned long long s1) {
    signed char bd[A];
    short legal[513];
    unsigned err = 0;
    for (int c = 0; c < A; c++) {
        const bool neg = (start[c >> 5] >> (c & 31)) & 1u, pos = (start[8 + (c >> 5)] >> (c & 31)) & 1u;
        bd[c] = pos ? 1 : (neg ? -1 : 0);
    }
    for (int k = 0; k < 513; k++) legal[k] = 0;
    EmuResult r = {0, 0u, 0u, 0u, 0ULL, 0ULL};
    int outcome = 2;
    for (;;) {
        if (r.plies >= 4096u) {
            err = 1;
            outcome = 0;
        }
        if (outcome != 2) break;
        if (legal[512] == 0) {  // legal_actions_playout_gomoku :196-207
            int count = 0;
            for (int c = 0; c < A; c++)
                if (bd[c] == 0) legal[count++] = (short)c;
            legal[512] = (short)count;
        }
        const int count = legal[512];
        const float u = rng_uniform_f32(s0, s1);
        const int ord = (int)(short)__float2int_rz(__fmul_rn(u, (float)count));
        if (u >= 1.0f) r.ub++;
        int action = legal[emu_wrap(ord, 513, err)];
        // take_action_playout_gomoku :210-217
        int i, j;
        if (action < 0) {
            err = 1;
            action = 0;
        }
        i = action / N;
        j = action % N;
        bd[emu_wrap(i, M, err) * N + emu_wrap(j, N, err)] = (signed char)turn;
        const int cnt = legal[512];
        const short last = legal[emu_wrap(cnt - 1, 513, err)];
        legal[emu_wrap(ord, 513, err)] = last;
        legal[512] = (short)(legal[512] - 1);
        turn = -turn;
        r.plies++;
        // compute_outcome_gomoku :220-281 (last_token = the stone just placed)
        const int token = -turn;
        const int di[4] = {1, 0, 1, 1}, dj[4] = {0, 1, 1, -1};
        outcome = 2;
        for (int d = 0; d < 4 && outcome == 2; d++) {
            int total = 0;
            for (int k = 1; k < 6; k++) {
                const int ii = i + k * di[d], jj = j + k * dj[d];
                if (ii < 0 || ii >= M || jj < 0 || jj >= N || bd[ii * N + jj] != token) break;
                total++;
            }
            for (int k = 1; k < 6; k++) {
                const int ii = i - k * di[d], jj = j - k * dj[d];
                if (ii < 0 || ii >= M || jj < 0 || jj >= N || bd[ii * N + jj] != token) break;
                total++;
            }
            if (total == 4) outcome = token;
        }
        if (outcome == 2) {
            bool draw = true;
            for (int c = 0; c < A; c++)
                if (bd[c] == 0) draw = false;
            if (draw) outcome = 0;
        }
    }
    r.outcome = outcome;
    r.err = err;
    r.s0 = s0;
    r.s1 = s1;
    return r;
}

__device__ __forceinline__ int turn_at_start(int mode, int sel_turn) { return mode == MODE_TREE_FULL ? sel_turn : -sel_turn; }

// ---------------------------------------------------------------------------------------------------------------
// The playouts, with games handed out to lanes one by one: a persistent grid of DYN_THREADS-thread blocks; every warp
// works through the games of one tree's step (game = active child * P + t, taken with one atomicAdd per refill by
// the warp's idle lanes together), then moves on to the next tree that still has games.  A lane that finishes its game
// waits until at least REFILL_MIN lanes of its warp are idle (a refill costs a few hundred instructions, mostly the copy
// of the legal-action list; doing it for several lanes at once keeps it a small fraction of the playing).  Which lane
// plays a game does not matter: game (child, t) draws from the stream of the reference's thread (tree, action, t).
// Per warp a copy of the parent position (Params::tpl) sits in shared memory; a child's list is the parent's without the
// child's own cell (the reference builds it by scanning the child's board in ascending order).
//
// Per-thread game state lives in shared memory, laid out so that every thread owns one bank column: word k of thread t
// is s_mem[k * DYN_THREADS + t].  That state (476 bytes) decides how many games an SM plays at once: two blocks of 224
// threads.  With so few warps the kernel is bound by the latency of a warp's own instruction chain, not by issue
// slots, which is what the choices below answer (Gomoku 15x15 acp_prodigal 4 x 256, 500 steps, one / eight searches,
// M playouts/s): a look at idle lanes after every ply 765 / 769, every 2nd 941 / 980, 4th 1004 / 1058, 8th 1053 / 1129
// (a lane whose game has ended sits out the plies up to the next look); refills for at least 4 idle lanes 1156 / 1429,
// 6: 1164 / 1485, 8: 1170 / 1500, 12: 1167 / 1478; blocks of 448 threads 1163 / 1434, of 128 threads (three per SM) slower.
#ifndef MCTSNC_GOMOKU_REFILL_MIN
#define MCTSNC_GOMOKU_REFILL_MIN 8
#endif
constexpr int REFILL_MIN = MCTSNC_GOMOKU_REFILL_MIN;
#ifndef MCTSNC_GOMOKU_PLIES_PER_LOOK
#define MCTSNC_GOMOKU_PLIES_PER_LOOK 8
#endif
constexpr int PLIES_PER_LOOK = MCTSNC_GOMOKU_PLIES_PER_LOOK;   // plies between two looks at whether lanes are idle
#ifndef MCTSNC_GOMOKU_UNROLL
#define MCTSNC_GOMOKU_UNROLL 8
#endif
constexpr int PLY_COPIES = MCTSNC_GOMOKU_UNROLL;   // copies of the ply's code in the loop between two looks
#ifndef MCTSNC_GOMOKU_THREADS
#define MCTSNC_GOMOKU_THREADS 224
#endif
constexpr int DYN_THREADS = MCTSNC_GOMOKU_THREADS;
// per warp: the parent position and, behind it, the ranks of the children that are played out (one byte each)
constexpr int WARP_ACTIVE = TPL_WORDS, WARP_WORDS = TPL_WORDS + 60;
constexpr size_t DYN_SMEM_BYTES = sizeof(unsigned) * ((size_t)THREAD_WORDS * DYN_THREADS + (size_t)WARP_WORDS * (DYN_THREADS / 32)) + FIVE_BYTES;
static_assert((THREAD_WORDS * DYN_THREADS) % 4 == 0 && WARP_WORDS % 4 == 0 && TPL_LINES % 4 == 0, "16-byte loads of the warp's copy");

// byte offset of list entry q of a thread from the thread's word 0: byte q & 3 of word q >> 2, words DYN_THREADS apart;
// (q >> 2) * 4 * DYN_THREADS + (q & 3) written as one shift and one multiply-add
__device__ __forceinline__ int list_byte(int q) { return (q >> 2) * (4 * DYN_THREADS - 4) + q; }

template <bool OCP>
__global__ void __launch_bounds__(DYN_THREADS) playout_dynamic_kernel(const Params p, int total_trees) {
    extern __shared__ __align__(16) unsigned s_mem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int P = p.n_playouts;
    int log2p = 0;
    while ((1 << log2p) < P) log2p++;
    unsigned *my = s_mem + tid;                                                     // word k of this thread: my[k * DYN_THREADS]
    unsigned *tpl = s_mem + THREAD_WORDS * DYN_THREADS + warp * WARP_WORDS;         // this warp's copy of the parent position
    const unsigned char *tpl_bytes = reinterpret_cast<const unsigned char *>(tpl + TPL_LIST);
    unsigned char *act_bytes = reinterpret_cast<unsigned char *>(tpl + WARP_ACTIVE);
    unsigned char *s_five = reinterpret_cast<unsigned char *>(s_mem + THREAD_WORDS * DYN_THREADS + WARP_WORDS * (DYN_THREADS / 32));
    for (int window = tid; window < FIVE_BYTES; window += DYN_THREADS) {
        int above = 0, below = 0;
        while (above < 5 && ((window >> (6 + above)) & 1)) above++;
        while (below < 5 && ((window >> (4 - below)) & 1)) below++;
        s_five[window] = above + below == 4 ? 1 : 0;
    }
    __syncthreads();
    int tree = p.tree_base + (int)(((long long)blockIdx.x * (DYN_THREADS / 32) + warp) % total_trees);
    int tried = 0;
    bool have_tpl = false, exhausted = false;
    // warp-uniform description of the current tree's step
    int n_items = 0, mode = 0, sel_turn = 0, count0 = 0, first_child = 0, selected = 0;
    // per-lane game (a lane may still be playing a game of an earlier tree after the warp has moved on)
    bool playing = false;
    int count = 0, turn = 0, action = 0, node = 0, my_tree = 0, my_start_turn = 0;
    int ord = 0;              // the draw of the ply to come, already turned into a position of the list
    int next_cell = 0, next_last = 0;   // list entries at that position and at the end of the list
    float count_2m64 = 0.f;   // count * 2^-64, the factor of the draws scaled by 2^64
    long long rng_idx = 0;
    unsigned long long s0 = 0, s1 = 0, start0 = 0, start1 = 0;
    unsigned plies = 0;
    for (;;) {
        if (!have_tpl) {
            // ---- describe the tree's step; fetch the parent position
            const StepInfo si = p.step[tree];
            mode = si.mode;
            n_items = si.n_active << log2p;
            selected = si.selected;
            first_child = si.first_child;
            sel_turn = g_turn(si.sel_meta);
            count0 = si.n_empty;
            int taken = 0;   // read by one lane, so that the whole warp sees the same value
            if (lane == 0) taken = *(volatile int *)&p.step[tree].game_counter;
            taken = __shfl_sync(0xFFFFFFFFu, taken, 0);
            exhausted = n_items == 0 || taken >= n_items;
            if (!exhausted) {
                __syncwarp();   // lanes of an earlier refill are done with the copy
                const unsigned *src = p.tpl + (long long)tree * TPL_WORDS;
                for (int w = lane; w < TPL_WORDS; w += 32) tpl[w] = src[w];
                const unsigned char *ranks = p.active_rank + tree * A;
                for (int k = lane; k < si.n_active; k += 32) act_bytes[k] = ranks[k];
                __syncwarp();
            }
            have_tpl = true;
        }
        // ---- refill: idle lanes take games together
        const unsigned idle = __ballot_sync(0xFFFFFFFFu, !playing);
        const int n_idle = __popc(idle);
        if (!exhausted && (n_idle >= REFILL_MIN || idle == 0xFFFFFFFFu) && n_idle > 0) {
            int base = 0;
            const int leader = __ffs(idle) - 1;
            if (lane == leader) base = atomicAdd(&p.step[tree].game_counter, n_idle);
            base = __shfl_sync(0xFFFFFFFFu, base, leader);
            if (base + n_idle >= n_items) exhausted = true;
            const int item = base + __popc(idle & ((1u << lane) - 1u));
            if (!playing && item < n_items) {
                const int t = item & (P - 1);
                int skip = 1 << 30;   // position of the parent's list that the child's list leaves out
                int cell = 0;
                if (mode == MODE_ALL_CHILDREN) {
                    const int rank = act_bytes[item >> log2p];
                    cell = tpl_bytes[rank];              // children are the first empty cells in ascending order
                    action = (cell >> 4) * N + (cell & 15);
                    skip = rank;
                    node = first_child + rank;
                    count = count0 - 1;
                    turn = -sel_turn;
                } else {   // the selected node itself is played out, with the streams of action 0
                    action = 0;
                    node = selected;
                    count = count0;
                    turn = sel_turn;
                }
                rng_idx = OCP ? ((long long)tree * P + t) : (((long long)tree * A + action) * P + t);
                const ulonglong2 rs = p.rng_playout[rng_idx];   // on its way while the position is copied
                // the child's list: the parent's without position `skip`.  Four words at a time; a word behind the one that
                // holds `skip` takes its bytes one position further up (a funnel shift by 0 or 8 bits), the word that holds
                // it is put right afterwards.  Words past the last entry are never read; up to three words past the list
                // are written and then covered by the lines.
                const int skip_word = skip >> 2;
                const int chunks = (count0 + 15) >> 4;
                const uint4 *tpl_list4 = reinterpret_cast<const uint4 *>(tpl + TPL_LIST);
                uint4 v = tpl_list4[0];
                for (int c = 0; c < chunks; c++) {
                    const uint4 nx = tpl_list4[c + 1];   // c + 1 <= 15: the lines follow the list in the warp's copy
                    const int d = skip_word - 4 * c;
                    unsigned *dst = my + 4 * c * DYN_THREADS;
                    dst[0 * DYN_THREADS] = __funnelshift_r(v.x, v.y, d < 0 ? 8 : 0);
                    dst[1 * DYN_THREADS] = __funnelshift_r(v.y, v.z, d < 1 ? 8 : 0);
                    dst[2 * DYN_THREADS] = __funnelshift_r(v.z, v.w, d < 2 ? 8 : 0);
                    dst[3 * DYN_THREADS] = __funnelshift_r(v.w, nx.x, d < 3 ? 8 : 0);
                    v = nx;
                }
                if (skip_word < LIST_WORDS) {
                    const unsigned prev = tpl[TPL_LIST + skip_word], next = tpl[TPL_LIST + skip_word + 1];
                    const unsigned keep = (1u << (8 * (skip & 3))) - 1u;
                    my[skip_word * DYN_THREADS] = (prev & keep) | (__funnelshift_r(prev, next, 8) & ~keep);
                }
                const uint4 *tpl_lines4 = reinterpret_cast<const uint4 *>(tpl + TPL_LINES);
#pragma unroll
                for (int c = 0; c < LINE_WORDS / 4; c++) {
                    const uint4 l = tpl_lines4[c];
                    unsigned *dst = my + (LIST_WORDS + 4 * c) * DYN_THREADS;
                    dst[0 * DYN_THREADS] = l.x;
                    dst[1 * DYN_THREADS] = l.y;
                    dst[2 * DYN_THREADS] = l.z;
                    dst[3 * DYN_THREADS] = l.w;
                }
                static_assert(LINE_WORDS % 4 == 2, "the last two line words");
                my[(LIST_WORDS + LINE_WORDS - 2) * DYN_THREADS] = tpl[TPL_LINES + LINE_WORDS - 2];
                my[(LIST_WORDS + LINE_WORDS - 1) * DYN_THREADS] = tpl[TPL_LINES + LINE_WORDS - 1];
                if (mode == MODE_ALL_CHILDREN) {   // the child's own stone, put down by the side to move at the parent
                    const int i = cell >> 4, j = cell & 15;
                    const int hs = sel_turn > 0 ? 16 : 0;
                    my[(LINE_ROW + i) * DYN_THREADS] |= 1u << (hs + j);
                    my[(LINE_COL + j) * DYN_THREADS] |= 1u << (hs + i);
                    my[(LINE_DIAG + ((i - j + 14) & 15)) * DYN_THREADS] |= 1u << (hs + j);
                    my[(LINE_ANTI + ((i + j) & 15)) * DYN_THREADS] |= 1u << (hs + j);
                }
                count_2m64 = (float)count * RNG_2M64;
                my_tree = tree;
                my_start_turn = turn;
                s0 = start0 = rs.x;
                s1 = start1 = rs.y;
                ord = __float2int_rz(__fmul_rn(rng_uniform_times_2p64(s0, s1), count_2m64));   // the draw of the first ply
                {
                    const unsigned char *list = reinterpret_cast<const unsigned char *>(my);
                    const int q_last = max(count - 1, 0);
                    next_last = list[list_byte(q_last)];
                    next_cell = list[list_byte(ord)];
                }
                plies = 0;
                playing = true;
            }
        }
        if (exhausted) {
            // ---- this tree's games are all taken: idle lanes take games of the next tree from now on, while the others
            // finish what they are playing (a game carries its tree with it); after the last tree the warp plays on until
            // its lanes are done
            if (tried + 1 < total_trees) {
                tried++;
                tree = tree + 1 == p.tree_base + total_trees ? p.tree_base : tree + 1;
                have_tpl = false;
                continue;
            }
            if (__ballot_sync(0xFFFFFFFFu, playing) == 0u) break;
        }
#pragma unroll(PLY_COPIES)
        for (int rep = 0; rep < PLIES_PER_LOOK; rep++) {
          if (playing) {
            // ---- one ply (src/mctsnc.py:2059-2064).  float32 u * int16 count -> float32 (:2061); here (u * 2^64) * (count * 2^-64):
            // the same product, rounded once.  u == 1.0f gives ord == count.  The draw of a ply is made one ply ahead, next to
            // the work of the ply before it, so that the chain of dependent steps of a ply starts at the list; if the game ends
            // with this ply, the stream is stored as it was before the draw for the next one.
            const int this_ord = ord;
            unsigned long long end0 = s0, end1 = s1;   // the stream after the draw of this ply
            ord = __float2int_rz(__fmul_rn(rng_uniform_times_2p64(s0, s1), count_2m64 - RNG_2M64));
            int outcome = 2;
            if (this_ord >= count) {
                // u == 1.0f: replay this game through the byte-level emulation of the reference
                const EmuResult er = playout_emulated(p.board + ((long long)my_tree * p.cap + node) * 16, my_start_turn, start0, start1);
                end0 = er.s0;
                end1 = er.s1;
                outcome = er.outcome;
                plies = er.plies;
                TreeState *st = p.state + my_tree;
                atomicAdd(&st->ub_draws, (unsigned long long)er.ub);
                atomicOr(&st->status, STATUS_UB_DRAW | (er.err ? STATUS_INTERNAL : 0u));
            } else {
                // last_action = legal[ord]; legal[ord] = legal[count - 1]; count -= 1   (:2062, :215-217).  List entry q of this
                // thread is byte q & 3 of its word q >> 2: byte loads and stores, no read-modify-write of words.  The two
                // entries a ply reads were fetched at the end of the ply before (after its store); here the two of the next
                // ply are fetched, so that they arrive while this ply's stone is tested.
                unsigned char *list = reinterpret_cast<unsigned char *>(my);
                const int cell = next_cell;
                list[list_byte(this_ord)] = (unsigned char)next_last;
                count--;
                count_2m64 -= RNG_2M64;   // exact: small integers times 2^-64
                const int q_last = max(count - 1, 0);
                next_last = list[list_byte(q_last)];
                next_cell = list[list_byte(ord)];   // ord <= count <= 225: inside the list words
                const int i = cell >> 4, j = cell & 15;
                const int hs = turn > 0 ? 16 : 0;
                plies++;
                // compute_outcome_gomoku (src/mctsnc_game_mechanics.py:220-272) without loops: the stone goes into the word of
                // its row, column, diagonal and anti-diagonal; of each word the mover's half is rotated so that the new
                // stone sits at bit 5, and the 11 bits around it index the table.  The bits of the half never wrap into the
                // window: rotating right by s = hs + pos - 5, a bit b < s lands at 32 - s + b >= 23 (low half: s <= 9; high
                // half: b >= 16, s <= 25), and a negative s is a shift of the low half to the left by at most 5.
                const unsigned half = 0x7FFFu << hs;
                const unsigned bit_j = 1u << (hs + j), bit_i = 1u << (hs + i);
                const int rot_j = hs + j - 5, rot_i = hs + i - 5;   // the funnel shift takes them modulo 32
                unsigned *row_w = my + (LINE_ROW + i) * DYN_THREADS;
                unsigned *col_w = my + (LINE_COL + j) * DYN_THREADS;
                unsigned *diag_w = my + (LINE_DIAG + ((i - j + 14) & 15)) * DYN_THREADS;
                unsigned *anti_w = my + (LINE_ANTI + ((i + j) & 15)) * DYN_THREADS;
                const unsigned wr = *row_w | bit_j, wc = *col_w | bit_i, wd = *diag_w | bit_j, wa = *anti_w | bit_j;
                *row_w = wr;
                *col_w = wc;
                *diag_w = wd;
                *anti_w = wa;
                const unsigned tr = wr & half, tc = wc & half, td = wd & half, ta = wa & half;
                const unsigned win = s_five[__funnelshift_r(tr, tr, rot_j) & 0x7FFu] | s_five[__funnelshift_r(tc, tc, rot_i) & 0x7FFu] |
                                     s_five[__funnelshift_r(td, td, rot_j) & 0x7FFu] | s_five[__funnelshift_r(ta, ta, rot_j) & 0x7FFu];
                if (win) outcome = turn;
                else if (count == 0) outcome = 0;
                turn = -turn;
            }
            if (outcome != 2) {
                p.rng_playout[rng_idx] = make_ulonglong2(end0, end1);
                if (outcome != 0) atomicAdd(&p.child_out[(my_tree * A + action) * 2 + (outcome > 0 ? 1 : 0)], 1);
                atomicAdd(&p.state[my_tree].plies, (unsigned long long)plies);
                playing = false;
            }
          }
        }
    }
}

}  // namespace gomoku
}  // namespace mctsnc
