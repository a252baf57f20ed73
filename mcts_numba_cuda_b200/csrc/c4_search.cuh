// Connect-4 search kernel: the whole MCTS-NC loop of one tree in one thread block, all steps on the device.
//
// Replaces, per step, the reference kernels _select (src/mctsnc.py:1293-1365), _expand_1_* (:1368-1681),
// _expand_2_* (:1691-1821), _playout_ocp / _playout_acp_* (:1824-2081), _backup_ocp / _backup_1_acp_* /
// _backup_2_acp (:2084-2220), the _reset kernel (:1260-1290) and the Connect-4 device functions
// (src/mctsnc_game_mechanics.py:89-179).
//
// Work split inside a block: warp 0 walks the tree (select), creates the children (expand) and writes the statistics
// back (backup); all threads play the random games.  A thread keeps playing its own list of games back to back (one
// per expanded child and playout index, the reference's thread (tree, action, t)), so the lanes of a warp wait for
// each other once per step, not once per game.
//
// Position encoding: column c of the 6x7 board owns bits 7c .. 7c+5 (bit 7c = bottom cell) and a guard bit 7c+6 that
// stays 0, so that shifts by 1, 6, 7, 8 test the four line directions without wrapping between columns.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "rng.cuh"

namespace mctsnc {
namespace c4 {

constexpr int ROWS = 6, COLS = 7, A = 7;
constexpr int LEGAL_SHIFT = 6;       // the playout loop keeps the set of open columns times 64 = byte offset of its row of move_lut
#ifndef MCTSNC_PLIES_PER_CHECK
#define MCTSNC_PLIES_PER_CHECK 4
#endif
constexpr int PLIES_PER_CHECK = MCTSNC_PLIES_PER_CHECK;  // plies of a playout between two looks at whether the game is over
constexpr unsigned long long BOTTOM_ROW = 0x0000040810204081ULL;  // bit 7c for c = 0..6
constexpr unsigned long long TOP_ROW = BOTTOM_ROW << 5;
constexpr unsigned long long FULL_BOARD = BOTTOM_ROW * 0x3FULL;
constexpr unsigned long long MOVE_LUT_NO_COLUMN = 1ULL << 63;

// four in a row anywhere in the stone set p.  Left shifts: the low word of a 64-bit left shift is a plain 32-bit
// shift, which the integer multiply-add pipe can execute, taking load off the logic pipe that limits this kernel.
// Bits shifted past bit 48 meet zeros of p in the AND.
__host__ __device__ __forceinline__ bool has_four(unsigned long long p) {
    unsigned long long m, r;
    m = p & (p << 7);
    r = m & (m << 14);
    m = p & (p << 6);
    r |= m & (m << 12);
    m = p & (p << 8);
    r |= m & (m << 16);
    m = p & (p << 1);
    r |= m & (m << 2);
    return r != 0;
}

// set of columns that still have room, from the occupancy bitboard
__host__ __device__ __forceinline__ unsigned legal_columns(unsigned long long all) {
    unsigned l = 0;
#pragma unroll
    for (int c = 0; c < COLS; c++) l |= ((all >> (7 * c + 5)) & 1ULL) ? 0u : (1u << c);
    return l;
}

// among tied maxima the reference's stride-halving reduction keeps the left operand (src/mctsnc.py:1343-1351), which
// over 8 slots ranks the actions 0,4,2,6,1,5,3 (smallest bit-reversed index wins)
__device__ __forceinline__ int pick_among_tied(unsigned m) {
    if (m & 1u) return 0;
    if (m & 16u) return 4;
    if (m & 4u) return 2;
    if (m & 64u) return 6;
    if (m & 2u) return 1;
    if (m & 32u) return 5;
    return 3;
}

__device__ __forceinline__ unsigned ordered_key(float v) {
    unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------------------------
// Byte-for-byte emulation of one playout of the reference (src/mctsnc.py:2049-2069 with the Connect-4 functions of
// src/mctsnc_game_mechanics.py:102-179) on int8 arrays.  Only entered when a uniform draw equals 1.0f, which makes
// the reference read legal_actions_with_count[count]: a value left by an earlier ply of the same playout, or a slot
// never written (read as 0 here).  numba wraps negative indices once; rows below 0 therefore address the board from
// the bottom.  The playout is replayed from its first ply so that the stale slots hold what they would hold.
struct EmuResult {
    int outcome;
    unsigned plies;
    unsigned ub;
    unsigned err;
    unsigned long long s0, s1;  // stream state after the game
};

__device__ __forceinline__ int emu_cell(const signed char *board, int i, int j, unsigned &err) {
    if (i < 0) i += ROWS;
    if (j < 0) j += COLS;
    if (i < 0 || i >= ROWS || j < 0 || j >= COLS) {
        err = 1;
        return 0;
    }
    return board[i * COLS + j];
}

__device__ __forceinline__ int emu_line(const signed char *board, int i, int j, int di, int dj, int token, unsigned &err) {
    int total = 0;
    for (int k = 1; k < 4; k++) {
        int ii = i + k * di, jj = j + k * dj;
        if ((di < 0 && ii < 0) || (di > 0 && ii >= ROWS) || (dj < 0 && jj < 0) || (dj > 0 && jj >= COLS)) break;
        if (emu_cell(board, ii, jj, err) != token) break;
        total++;
    }
    return total;
}

__device__ __noinline__ EmuResult playout_emulated(unsigned long long neg, unsigned long long pos, int turn,
                                                   unsigned long long s0, unsigned long long s1) {
    unsigned err = 0;
    signed char board[ROWS * COLS];
    signed char fills[COLS];
    short legal[COLS + 1];
    for (int j = 0; j < COLS; j++) {
        int f = 0;
        for (int h = 0; h < ROWS; h++) {
            int bit = 7 * j + h;
            int v = ((pos >> bit) & 1ULL) ? 1 : (((neg >> bit) & 1ULL) ? -1 : 0);
            board[(ROWS - 1 - h) * COLS + j] = (signed char)v;
            f += v != 0;
        }
        fills[j] = (signed char)f;
    }
    for (int j = 0; j <= COLS; j++) legal[j] = 0;
    EmuResult r = {2, 0u, 0u, 0u, 0ULL, 0ULL};
    for (;;) {
        int count = 0;
        for (int j = 0; j < COLS; j++)
            if (fills[j] < ROWS) legal[count++] = (short)j;
        float u = rng_uniform_f32(s0, s1);
        int ord = (int)(short)__float2int_rz(__fmul_rn(u, (float)count));
        if (u >= 1.0f) r.ub++;
        if (ord < 0 || ord > COLS) {
            err = 1;
            ord = 0;
        }
        int a = legal[ord];
        fills[a] += 1;
        int row = ROWS - fills[a];
        if (row < 0) row += ROWS;
        if (row < 0) {
            err = 1;
            row = 0;
        }
        board[row * COLS + a] = (signed char)turn;
        turn = -turn;
        r.plies++;
        // compute_outcome_c4(board, fills, turn, a)
        int token = -turn;
        int i = ROWS - fills[a];
        int out = 2;
        if (emu_line(board, i, a, -1, 0, token, err) + emu_line(board, i, a, 1, 0, token, err) >= 3) out = token;
        else if (emu_line(board, i, a, 0, 1, token, err) + emu_line(board, i, a, 0, -1, token, err) >= 3) out = token;
        else if (emu_line(board, i, a, -1, 1, token, err) + emu_line(board, i, a, 1, -1, token, err) >= 3) out = token;
        else if (emu_line(board, i, a, -1, -1, token, err) + emu_line(board, i, a, 1, 1, token, err) >= 3) out = token;
        else {
            bool draw = true;
            for (int j = 0; j < COLS; j++)
                if (fills[j] < ROWS) draw = false;
            if (draw) out = 0;
        }
        if (r.plies > 4096u) {  // cannot happen; keeps the loop bounded whatever the memory holds
            err = 1;
            out = 0;
        }
        if (out != 2) {
            r.outcome = out;
            r.err = err;
            r.s0 = s0;
            r.s1 = s1;
            return r;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------

// everything a thread needs to start a game from one child, fetched with two 16-byte shared-memory loads
struct __align__(16) GameSlot {
    unsigned long long cur;  // stones of the side to move
    unsigned long long top;  // one bit per column: its lowest empty cell (the guard bit of a full column) = all stones + BOTTOM_ROW
    unsigned legal;          // columns with room, shifted left by LEGAL_SHIFT
    int rng_base;            // index of the child's first stream in the block's stream array
    int stones;              // stones on the board
    float count;             // number of columns with room times 2^-64 (the playout loop draws uniforms scaled by 2^64)
};

struct Shared {
    GameSlot slot[A];        // children that need real playouts, in expansion order
    int tally[A][2];         // per slot: games won by -1, by +1 (of the games this block played)
    int gather[A][2];        // cluster of blocks per tree: the sums over the blocks, kept by the first block
    int path[48];
    int path_ns[48];
    int path_wins[48];
    int child_action[A];     // per expanded child (expansion order): its action,
    int child_outcome[A];    // its outcome (2 = ongoing)
    int child_slot[A];       // and its slot (-1: no playouts: terminal, or not picked in OCP)
    int child_out[A][2];     // trees_playout_outcomes_children (persists over steps)
    short ae[A + 2];         // trees_actions_expanded row (persists over steps)
    // move_lut[set * 8 + ord]: for the ord-th column (ascending) of the column set `set`, the six cells of the column
    // (0x3F << 7 * column) in bits 0..47 and the column's bit in bits 54..60, i.e. where it sits in the pre-shifted column
    // set the playout loop keeps (GameSlot::legal), moved up by 48.  An ordinal the set does not have (only a uniform
    // draw of exactly 1.0f gives one: ord == number of columns) maps to MOVE_LUT_NO_COLUMN: no cell, bit 63 set.
    unsigned long long move_lut[128 * 8];
    int job;                 // tree of the slice being run (-1: none left)
    int n_slots;
    int next_item;           // next game to hand out in the playout phase
    int n_exp;
    int mode;
    int first_child;
    int exp_mask;
    int selected;
    int sel_meta;
    int path_len;
    int pick;                // OCP: index (among expanded children) of the child that is played out
    int root_turn;
    int size;
    int out_neg, out_pos;
    unsigned status;
    unsigned long long plies;
    unsigned long long ub;
    unsigned long long stage_cycles[4];  // cycles of this slice spent in select, expand, playouts, backup (thread 0 keeps them)
    unsigned stage_mark;        // cycle counter when the playouts of the current step began
};

// Node records through the copy the walker keeps of a tree's first `cache_n` records (cluster kernel: the walk down the tree
// is a chain of dependent loads, and the upper levels of a tree are its oldest nodes); cache_n = 0: global memory only.
// Every store goes to both.
__device__ __forceinline__ int4 rec_load(const int4 *rec, const int4 *cache, int cache_n, int i) {
    return i < cache_n ? cache[i] : rec[i];
}
__device__ __forceinline__ void rec_store(int4 *rec, int4 *cache, int cache_n, int i, int4 v) {
    rec[i] = v;
    if (i < cache_n) cache[i] = v;
}
__device__ __forceinline__ void rec_store_stats(int4 *rec, int4 *cache, int cache_n, int i, int ns, int wins) {
    *reinterpret_cast<int2 *>(&rec[i]) = make_int2(ns, wins);
    if (i < cache_n) *reinterpret_cast<int2 *>(&cache[i]) = make_int2(ns, wins);
}

// `n_steps` steps of tree g by the whole block, from the state the tree has in global memory and back to it.
// The random streams of the tree (ACP: 7*P, OCP: P states of 16 B) stay in dynamic shared memory meanwhile: they are
// read at the start of every game and written back at its end, by one thread each.
//
// CL > 1: a thread-block cluster of CL blocks grows the tree (launches with so few trees that a tree would otherwise be
// bound by what one SM can play per step).  The first block of the cluster walks, expands and backs up as before and
// hands the step's games (slots) to the shared memory of the others; every block plays the games of P / CL of the P
// playout indices of every child -- it keeps the streams of exactly those in its shared memory -- and adds its tallies
// to the first block's `gather`.  Two cluster barriers per step; all blocks run the same loop, so every block reaches
// every barrier.
template <bool OCP, int CL>
__device__ __forceinline__ void run_slice(const SearchParams &p, Shared &s, ulonglong2 *s_rng, int4 *cache, const int g,
                                          const int n_steps, const bool first) {
    namespace cg = cooperative_groups;
    const int cache_n = CL > 1 ? p.cache_nodes : 0;
    static_assert(CL == 1 || CL == 2 || CL == 4 || CL == 8, "cluster sizes");
    constexpr int LOG_CL = CL == 8 ? 3 : (CL == 4 ? 2 : (CL == 2 ? 1 : 0));
    const int tid = threadIdx.x;
    const int nt = blockDim.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int P = p.n_playouts;
    const int rank = CL > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int log2_local = p.log2_playouts - LOG_CL;   // this block plays P_local = P / CL playout indices of every child
    const int P_local = P >> LOG_CL;
    int4 *rec = p.rec + (long long)g * p.cap;
    ulonglong2 *board = p.board + (long long)g * p.cap;
    int *parent = p.parent + (long long)g * p.cap;
    TreeState *st = p.state + g;
    const bool thrifty = (p.variant == 0 || p.variant == 2);
    const bool walker = warp == 0 && rank == 0;   // the warp that selects, expands and backs up

    const int n_streams = OCP ? P : A * P;
    ulonglong2 *g_rng = p.rng_playout + (long long)g * n_streams;
    // stream (action, t) of the tree sits at local index action * P_local + (t - rank * P_local)
    for (int i = tid; i < (n_streams >> LOG_CL); i += nt)
        s_rng[i] = g_rng[((i >> log2_local) << p.log2_playouts) + rank * P_local + (i & (P_local - 1))];
    if (CL > 1 && tid < 2 * A) s.tally[tid >> 1][tid & 1] = 0;
    if (tid == 0 && rank == 0) {
        const int b = g / p.n_trees;
        if (first) {
            const int turn = p.root_turn[b];
            rec_store(rec, cache, cache_n, 0, make_int4(0, 0, -1, make_meta(0, false, 2, turn, 0)));
            board[0] = p.root_board[b];
            parent[0] = -1;
            s.size = 1;
            s.root_turn = turn;
            s.status = 0;
            s.plies = 0;
            s.ub = 0;
            s.selected = 0;
            s.path_len = 1;
        } else {
            s.size = st->size;
            s.root_turn = meta_turn(rec[0].w);
            s.status = st->status;
            s.plies = st->plies;
            s.ub = st->ub_draws;
            s.selected = st->selected;
            s.path_len = st->path_len;
        }
        for (int k = 0; k < 4; k++) s.stage_cycles[k] = 0;
        // the "last step" arrays of the reference live as long as the instance: a new search starts from what the
        // previous one left in them (trees_actions_expanded keeps stale entries in the thrifty layout)
        s.out_neg = st->out_neg;
        s.out_pos = st->out_pos;
        for (int a = 0; a < A; a++) {
            s.child_out[a][0] = p.child_out[(g * A + a) * 2 + 0];
            s.child_out[a][1] = p.child_out[(g * A + a) * 2 + 1];
        }
        for (int a = 0; a < A + 2; a++) s.ae[a] = p.actions_expanded[g * (A + 2) + a];
    }
    if (CL > 1) cg::this_cluster().sync();
    else __syncthreads();
    if (CL > 1 && rank == 0 && !first) {   // a search that goes on: the records the tree has so far
        const int have = s.size < cache_n ? s.size : cache_n;
        for (int i = tid; i < have; i += nt) cache[i] = rec[i];
        __syncthreads();
    }

    const double c_ucb = (double)p.ucb_c;
    unsigned my_plies = 0, my_ub = 0, my_err = 0;

    // The walker warp runs steps on its own for as long as they select a terminal node (nothing to play: the backup follows
    // at once) and meets the other threads only for a step with games, or when the steps are done (MODE_DONE).
    int step = 0;
    bool backup_due = false;   // the walker's: the step it selected last has not been backed up yet
    for (;;) {
        // =========================================================== backup of the step before, select + expand (warp 0)
        if (walker) for (;;) {
            if (backup_due) {
                // ======================================================= backup (_backup_* of the reference)
                __syncwarp();
                const unsigned c_backup = (unsigned)clock();
                const int (*tally)[2] = CL > 1 ? s.gather : s.tally;
                const int mode = s.mode;
                const int n_exp = s.n_exp;
                const int sel_meta = s.sel_meta;
                const int child_turn = -meta_turn(sel_meta);
                int neg_tot = 0, pos_tot = 0;
                long long n_tot = P;
                if (mode == MODE_ALL_CHILDREN) {
                    int my_neg = 0, my_pos = 0;
                    if (lane < n_exp) {
                        const int o = s.child_outcome[lane];
                        const int j = s.child_slot[lane];
                        const bool played = !OCP || lane == s.pick;
                        if (j >= 0) {
                            my_neg = tally[j][0];
                            my_pos = tally[j][1];
                        } else if (played) {
                            // a terminal child: its stored outcome stands for all P playouts (src/mctsnc.py:2016-2021)
                            my_neg = o == -1 ? P : 0;
                            my_pos = o == 1 ? P : 0;
                        }
                        // children start from ns = ns_wins = 0 (src/mctsnc.py:1819-1820), then _backup_1_acp_* / the
                        // thread-0 part of _backup_ocp credit them (:2172-2177, :2104-2114)
                        const int cns = played ? P : 0;
                        const int cw = played ? (child_turn == 1 ? my_neg : my_pos) : 0;
                        rec_store(rec, cache, cache_n, s.first_child + lane,
                                  make_int4(cns, cw, -1, make_meta(0, o != 2, o, child_turn, meta_depth(sel_meta) + 1)));
                        if (!OCP) {
                            s.child_out[s.child_action[lane]][0] = my_neg;
                            s.child_out[s.child_action[lane]][1] = my_pos;
                        }
                    }
                    neg_tot = __reduce_add_sync(0xFFFFFFFFu, my_neg);
                    pos_tot = __reduce_add_sync(0xFFFFFFFFu, my_pos);
                    if (!OCP) n_tot = (long long)P * n_exp;
                } else if (mode == MODE_TERMINAL) {
                    neg_tot = s.out_neg;
                    pos_tot = s.out_pos;
                } else {
                    neg_tot = tally[0][0];
                    pos_tot = tally[0][1];
                    if (!OCP && lane == 0) {
                        s.child_out[0][0] = neg_tot;
                        s.child_out[0][1] = pos_tot;
                    }
                }
                const int plen = s.path_len;
                for (int e = lane; e < plen; e += 32) {
                    const int node = s.path[e];
                    const int turn_e = (e & 1) ? -s.root_turn : s.root_turn;
                    const int ns = s.path_ns[e] + (int)n_tot;
                    const int wins = s.path_wins[e] + (turn_e == 1 ? neg_tot : pos_tot);
                    if (e == plen - 1 && mode == MODE_ALL_CHILDREN) {
                        rec_store(rec, cache, cache_n, node, make_int4(ns, wins, s.first_child, sel_meta | s.exp_mask));
                    } else {
                        rec_store_stats(rec, cache, cache_n, node, ns, wins);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    s.out_neg = neg_tot;
                    s.out_pos = pos_tot;
                    s.stage_cycles[2] += c_backup - s.stage_mark;
                    s.stage_cycles[3] += (unsigned)clock() - c_backup;
                }
                __syncwarp();
                backup_due = false;
            }
            if (step == n_steps) {
                if (lane == 0) s.mode = MODE_DONE;
                if (CL > 1 && lane > 0 && lane < CL) cg::this_cluster().map_shared_rank(&s, lane)->mode = MODE_DONE;
                break;
            }
            const unsigned c_step = (unsigned)clock();   // 32-bit cycle counts: differences are right modulo 2^32
            int node = 0;
            int4 r = rec_load(rec, cache, cache_n, 0);
            int depth = 0;
            if (lane == 0) {
                s.path[0] = 0;
                s.path_ns[0] = r.x;
                s.path_wins[0] = r.y;
            }
            // log(N) of the node being left is needed by every child's UCB; each lane computes the logarithm of ITS child's
            // count while it evaluates the child's UCB (two independent float64 chains), so the winner's value is ready
            // for the next level instead of starting that level with a ~100-operation dependent chain
            double log_parent = (r.w & 0x7F) != 0 ? log((double)r.x) : 0.0;
            while ((r.w & 0x7F) != 0 && depth < 46) {
                const unsigned mask = r.w & 0x7F;
                int child = -1;
                int4 cr = make_int4(0, 0, -1, 0);
                unsigned key = 0;
                double log_child = 0.0;
                if (lane < A && ((mask >> lane) & 1u)) {
                    child = r.z + __popc(mask & ((1u << lane) - 1u));
                    cr = rec_load(rec, cache, cache_n, child);
                    float v;
                    if (cr.x == 0) {
                        v = __int_as_float(0x7f800000);
                    } else {
                        // src/mctsnc.py:1337 -- evaluated in float64 (numba promotes int32/float32 and log(int32) to
                        // float64), fused multiply-add as NVVM contracts it, rounded once to float32
                        const double q = (double)cr.y / (double)__int2float_rn(cr.x);
                        const double e = sqrt(log_parent / (double)cr.x);
                        v = __double2float_rn(fma(c_ucb, e, q));
                        log_child = log((double)cr.x);
                    }
                    key = ordered_key(v);
                }
                const unsigned best = __reduce_max_sync(0xFFFFFFFFu, key);
                const unsigned tied = __ballot_sync(0xFFFFFFFFu, key == best && child >= 0) & 0x7Fu;
                const int w = pick_among_tied(tied);
                node = __shfl_sync(0xFFFFFFFFu, child, w);
                r.x = __shfl_sync(0xFFFFFFFFu, cr.x, w);
                r.y = __shfl_sync(0xFFFFFFFFu, cr.y, w);
                r.z = __shfl_sync(0xFFFFFFFFu, cr.z, w);
                r.w = __shfl_sync(0xFFFFFFFFu, cr.w, w);
                log_parent = __shfl_sync(0xFFFFFFFFu, log_child, w);
                depth++;
                if (lane == 0) {
                    s.path[depth] = node;
                    s.path_ns[depth] = r.x;
                    s.path_wins[depth] = r.y;
                }
            }
            // ------------------------------------------------------- expand (_expand_1_* and _expand_2_*)
            const unsigned c_expand = (unsigned)clock();
            const int sel_turn = meta_turn(r.w);
            int mode, n_exp = 0, exp_mask = 0, first_child = -1, pick = 0, n_slots = 0;
            if (r.w & META_TERMINAL) {
                mode = MODE_TERMINAL;
                if (lane == 0) {
                    const int o = meta_outcome(r.w);
                    s.out_neg = o == -1 ? P : 0;
                    s.out_pos = o == 1 ? P : 0;
                }
            } else {
                const ulonglong2 bb = board[node];  // x: stones of -1, y: stones of +1
                const unsigned long long all = bb.x | bb.y;
                const unsigned legal = legal_columns(all);
                const int n_legal = __popc(legal);
                long long room = p.node_limit - (long long)s.size;
                if (room < 0) room = 0;
                n_exp = n_legal < room ? n_legal : (int)room;
                exp_mask = (int)legal;
                for (int drop = n_legal - n_exp; drop > 0; drop--)  // keep the n_exp lowest legal actions
                    exp_mask &= ~(1 << (31 - __clz(exp_mask)));
                if (n_exp < n_legal && lane == 0) s.status |= STATUS_TREE_FULL;
                if (n_exp > 0) {
                    mode = MODE_ALL_CHILDREN;
                    first_child = s.size;
                    if (OCP) {
                        // src/mctsnc.py:1435 / :1511 -- float32 * int64 is a float64 product, truncated
                        if (lane == 0) {
                            ulonglong2 es = p.rng_expand[g];
                            const float u = rng_uniform_f32(es.x, es.y);
                            p.rng_expand[g] = es;
                            pick = __double2int_rz((double)u * (double)n_exp);
                            if (pick >= n_exp) {  // u == 1.0f: undefined in the reference, clamped
                                pick = n_exp - 1;
                                s.ub++;
                                s.status |= STATUS_UB_DRAW;
                            }
                        }
                        pick = __shfl_sync(0xFFFFFFFFu, pick, 0);
                    }
                    const bool has_child = lane < A && ((exp_mask >> lane) & 1);
                    const int k = __popc(exp_mask & ((1 << lane) - 1));
                    unsigned long long cneg = bb.x, cpos = bb.y, call = all;
                    int outcome = 2;
                    if (has_child) {
                        const unsigned long long move = (all + (1ULL << (7 * lane))) & (0x3FULL << (7 * lane));
                        if (sel_turn > 0) cpos |= move;
                        else cneg |= move;
                        call = all | move;
                        const bool win = has_four(sel_turn > 0 ? cpos : cneg);
                        outcome = win ? sel_turn : (call == FULL_BOARD ? 0 : 2);
                        board[first_child + k] = make_ulonglong2(cneg, cpos);
                        parent[first_child + k] = node;
                    }
                    const bool plays = has_child && outcome == 2 && (!OCP || k == pick);
                    const unsigned play_mask = __ballot_sync(0xFFFFFFFFu, plays);
                    n_slots = __popc(play_mask);
                    if (has_child) {
                        const int j = plays ? __popc(play_mask & ((1u << lane) - 1u)) : -1;
                        s.child_action[k] = lane;
                        s.child_outcome[k] = outcome;
                        s.child_slot[k] = j;
                        if (plays) {
                            GameSlot gs;
                            gs.cur = sel_turn > 0 ? cneg : cpos;  // the child is to be moved in by the other side
                            gs.top = call + BOTTOM_ROW;
                            gs.legal = legal_columns(call) << LEGAL_SHIFT;
                            gs.rng_base = OCP ? 0 : lane * P;
                            gs.stones = __popcll(call);
                            gs.count = (float)__popc(gs.legal) * RNG_2M64;
                            s.slot[j] = gs;
                            s.tally[j][0] = 0;
                            s.tally[j][1] = 0;
                            s.gather[j][0] = 0;
                            s.gather[j][1] = 0;
                        }
                    }
                } else {
                    // no room for a single child: the selected node itself is played out
                    mode = MODE_TREE_FULL;
                    n_slots = 1;
                    if (lane == 0) {
                        GameSlot gs;
                        gs.cur = sel_turn > 0 ? bb.y : bb.x;
                        gs.top = all + BOTTOM_ROW;
                        gs.legal = legal << LEGAL_SHIFT;
                        gs.rng_base = 0;
                        gs.stones = __popcll(all);
                        gs.count = (float)n_legal * RNG_2M64;
                        s.slot[0] = gs;
                        s.tally[0][0] = 0;
                        s.tally[0][1] = 0;
                        s.gather[0][0] = 0;
                        s.gather[0][1] = 0;
                    }
                }
            }
            // trees_actions_expanded in the layout of the variant (src/mctsnc.py:1430-1454, :1509-1531, :1583-1604,
            // :1656-1681)
            if (lane < A) {
                if (thrifty) {
                    if (mode == MODE_ALL_CHILDREN && ((exp_mask >> lane) & 1))
                        s.ae[__popc(exp_mask & ((1 << lane) - 1))] = (short)lane;
                } else {
                    if (mode == MODE_ALL_CHILDREN) s.ae[lane] = ((exp_mask >> lane) & 1) ? (short)lane : (short)-1;
                    else s.ae[lane] = -1;
                }
            }
            __syncwarp();
            if (lane == 0) {
                if (mode == MODE_ALL_CHILDREN) s.size += n_exp;
                s.ae[A + 1] = (short)(mode == MODE_ALL_CHILDREN ? n_exp : 1);
                int m2 = mode;
                if (OCP && mode == MODE_ALL_CHILDREN) m2 = thrifty ? pick : s.child_action[pick];
                s.ae[A] = (short)m2;
                if (!OCP && mode != MODE_ALL_CHILDREN) s.ae[0] = 0;
                s.next_item = 0;
                s.n_slots = n_slots;
                s.pick = pick;
                s.mode = mode;
                s.n_exp = n_exp;
                s.exp_mask = exp_mask;
                s.first_child = first_child;
                s.selected = node;
                s.sel_meta = r.w;
                s.path_len = depth + 1;
                const unsigned c_play = (unsigned)clock();
                s.stage_cycles[0] += c_expand - c_step;
                s.stage_cycles[1] += c_play - c_expand;
                s.stage_mark = c_play;
            }
            step++;
            backup_due = true;
            if (mode == MODE_TERMINAL) continue;
            if (CL > 1) {
                // the step's games for the other blocks of the cluster: stores into their shared memory, made visible by
                // the barrier below
                __syncwarp();
                for (int other = 1; other < CL; other++) {
                    Shared *rs = cg::this_cluster().map_shared_rank(&s, other);
                    if (lane < n_slots) rs->slot[lane] = s.slot[lane];
                    if (lane == 0) {
                        rs->n_slots = n_slots;
                        rs->mode = mode;
                        rs->sel_meta = r.w;
                        rs->next_item = 0;
                    }
                }
            }
            break;
        }
        if (CL > 1) cg::this_cluster().sync();
        else __syncthreads();
        if (s.mode == MODE_DONE) break;

        // =========================================================== playouts (all threads)
        // Games are handed out one at a time from a counter in shared memory, so the threads of the block stay busy
        // until the step's games run out whatever their lengths.  Game `item` is playout t = item % P of slot
        // item / P; it draws from the stream the reference's thread (tree, action, t) owns (src/mctsnc.py:1938, :2028;
        // OCP: cuda.grid(1), :1849), so which thread plays it does not matter.
        //
        // The board of a game in progress is three words: the stones of the side that moves at the even plies of a
        // block of PLIES_PER_CHECK plies (a game starts at ply 0 of a block, so that is the side to move in the game's
        // first position), the stones of the other side, and `top`, one bit per column at its lowest empty cell (the
        // guard bit once the column is full; top = all stones + BOTTOM_ROW).  A move in a column with room is then
        // top & (six cells of the column), and top + move puts the marker one cell up.
        {
            const int n_items = s.n_slots << log2_local;
            // the side to move in the played-out positions: the other side than at the selected node, unless the
            // selected node itself is played out
            const int first_mover = (s.mode == MODE_TREE_FULL) ? meta_turn(s.sel_meta) : -meta_turn(s.sel_meta);
            unsigned long long side_even = 0, side_odd = 0, top = 0, s0 = 0, s1 = 0;
            unsigned legal = 0;
            float count = 0.f;
            int rng_idx = 0, stones = 0, j = 0;
            int item = atomicAdd(&s.next_item, 1);
            if (item < n_items) {
                j = item >> log2_local;
                const GameSlot gs = s.slot[j];
                side_even = gs.cur;
                side_odd = (gs.top - BOTTOM_ROW) ^ gs.cur;
                top = gs.top;
                legal = gs.legal;
                count = gs.count;
                stones = gs.stones;
                rng_idx = (gs.rng_base >> LOG_CL) + (item & (P_local - 1));
                const ulonglong2 rs = s_rng[rng_idx];
                s0 = rs.x;
                s1 = rs.y;
            }
            while (item < n_items) {
                // A finished game is noticed only every PLIES_PER_CHECK plies: its lane sits out the plies in between.  The
                // code that closes a game and fetches the next one (about 30 instructions) runs for the few lanes whose
                // games have just ended while the others wait, and with a check after every ply it ran in nearly every
                // iteration; checking after every fourth ply costs a little lane time and saved 10 % of the run time
                // (13.8 -> 15.3 G playouts/s on the headline workload; 2: 14.9, 3: 15.3, 5: 15.4, 8: 14.1).
                bool win = false, over = false;
                unsigned no_column = 0;   // bit 31 set once a draw of 1.0f asked for a column the position does not have
                static_assert(PLIES_PER_CHECK % 2 == 0, "the two sides alternate by the parity of the ply within a block");
#pragma unroll
                for (int k = 0; k < PLIES_PER_CHECK; k++) {
                    if (over) continue;
                    // ---- one ply (src/mctsnc.py:2059-2064, :2069)
                    // float32 u * int16 count -> float32 (:2061); here (u * 2^64) * (count * 2^-64): the same product.
                    // u == 1.0f gives ord == count, which the table answers with MOVE_LUT_NO_COLUMN: nothing is played, the flag
                    // sticks, and the game is replayed from its start through the byte-level emulation when it is closed
                    const float f = rng_uniform_times_2p64(s0, s1);
                    const int ord = __float2int_rz(__fmul_rn(f, count));
                    const unsigned long long e = *reinterpret_cast<const unsigned long long *>(
                        reinterpret_cast<const char *>(s.move_lut) + (legal + ord * 8));
                    no_column |= (unsigned)(e >> 32);
                    const unsigned long long move = top & e;
                    top += move;
                    // the sides take turns with the plies of the unrolled block: no swap of "mine" and "theirs"
                    unsigned long long mine;
                    if (k & 1) {
                        side_odd |= move;
                        mine = side_odd;
                    } else {
                        side_even |= move;
                        mine = side_even;
                    }
                    win = has_four(mine);
                    if ((move & TOP_ROW) != 0) {
                        legal ^= (unsigned)(e >> 48);
                        count -= RNG_2M64;
                    }
                    over = win || count == 0.0f;
                }
                if (over || (no_column & 0x80000000u)) {
                    int n = __popcll(side_even | side_odd) - stones;  // plies of this game; the last one was made by the
                    int winner = 0;                                    // first mover iff n is odd
                    if (win) winner = (n & 1) ? first_mover : -first_mover;
                    if (no_column & 0x80000000u) {
                        // u == 1.0f somewhere in this game: replay it through the byte-level emulation of the reference
                        const GameSlot gs = s.slot[j];
                        const ulonglong2 rs = s_rng[rng_idx];
                        const unsigned long long other = (gs.top - BOTTOM_ROW) ^ gs.cur;
                        const EmuResult er = playout_emulated(first_mover > 0 ? other : gs.cur, first_mover > 0 ? gs.cur : other,
                                                              first_mover, rs.x, rs.y);
                        s0 = er.s0;
                        s1 = er.s1;
                        winner = er.outcome == 2 ? 0 : er.outcome;
                        n = (int)er.plies;
                        my_ub += er.ub;
                        my_err |= er.err;
                    }
                    s_rng[rng_idx] = make_ulonglong2(s0, s1);
                    my_plies += n;
                    if (winner != 0) atomicAdd(&s.tally[j][winner > 0 ? 1 : 0], 1);
                    item = atomicAdd(&s.next_item, 1);
                    if (item < n_items) {
                        j = item >> log2_local;
                        const GameSlot gs = s.slot[j];
                        side_even = gs.cur;
                        side_odd = (gs.top - BOTTOM_ROW) ^ gs.cur;
                        top = gs.top;
                        legal = gs.legal;
                        count = gs.count;
                        stones = gs.stones;
                        rng_idx = (gs.rng_base >> LOG_CL) + (item & (P_local - 1));
                        const ulonglong2 rs = s_rng[rng_idx];
                        s0 = rs.x;
                        s1 = rs.y;
                    }
                }
            }
        }
        if (CL > 1) {
            // this block's tallies go to the first block's sums (atomic adds into its shared memory), then start from zero
            __syncthreads();
            if (tid < 2 * A) {
                const int v = s.tally[tid >> 1][tid & 1];
                if (v != 0) {
                    atomicAdd(&cg::this_cluster().map_shared_rank(&s, 0)->gather[tid >> 1][tid & 1], v);
                    s.tally[tid >> 1][tid & 1] = 0;
                }
            }
            cg::this_cluster().sync();
        } else {
            __syncthreads();
        }
    }

    // =============================================================== leave the per-tree state for the next launch
    {
        Shared *home = CL > 1 ? cg::this_cluster().map_shared_rank(&s, 0) : &s;   // the first block keeps the tree's counters
        if (my_plies) atomicAdd(&home->plies, (unsigned long long)my_plies);
        if (my_ub) {
            atomicAdd(&home->ub, (unsigned long long)my_ub);
            atomicOr(&home->status, STATUS_UB_DRAW);
        }
        if (my_err) atomicOr(&home->status, STATUS_INTERNAL);
    }
    if (CL > 1) cg::this_cluster().sync();   // also: no block leaves while another may still write to its shared memory
    else __syncthreads();
    for (int i = tid; i < (n_streams >> LOG_CL); i += nt)
        g_rng[((i >> log2_local) << p.log2_playouts) + rank * P_local + (i & (P_local - 1))] = s_rng[i];
    if (rank != 0) return;
    if (tid == 0) {
        st->size = s.size;
        st->selected = s.selected;
        st->path_len = s.path_len;
        st->out_neg = s.out_neg;
        st->out_pos = s.out_pos;
        st->status = s.status;
        st->plies = s.plies;
        st->ub_draws = s.ub;
        for (int k = 0; k < 4; k++) st->stage_ms[k] = (first ? 0.f : st->stage_ms[k]) + (float)s.stage_cycles[k] * p.ms_per_cycle;
        for (int a = 0; a < A; a++) {
            p.child_out[(g * A + a) * 2 + 0] = s.child_out[a][0];
            p.child_out[(g * A + a) * 2 + 1] = s.child_out[a][1];
        }
        for (int a = 0; a < A + 2; a++) p.actions_expanded[g * (A + 2) + a] = s.ae[a];
        for (int e = 0; e < s.path_len; e++) p.paths[g * PATH_CAP + e] = s.path[e];
    }
}

// One block grows one tree at a time.  Without a queue block b runs the whole launch of tree b.  With a queue (batched
// launches with more trees than blocks fit on the device) the grid is persistent and the blocks take slices of
// p.chunk steps of whichever tree is next in the ring.
__device__ __forceinline__ long long global_timer_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void build_move_lut(Shared &s) {
    for (int i = threadIdx.x; i < 128 * 8; i += blockDim.x) {
        const int set = i >> 3, ord = i & 7;
        int col = -1, seen = 0;
        for (int c = 0; c < COLS; c++)
            if (set & (1 << c)) {
                if (seen == ord) col = c;
                seen++;
            }
        s.move_lut[i] = col < 0 ? MOVE_LUT_NO_COLUMN
                                : (0x3FULL << (7 * col)) | ((unsigned long long)((1 << col) << LEGAL_SHIFT) << 48);
    }
}

#ifndef MCTSNC_C4_MAXNREG
#define MCTSNC_C4_MAXNREG 64
#endif
template <bool OCP>
__global__ void __maxnreg__(MCTSNC_C4_MAXNREG) search_kernel(const SearchParams p) {
    __shared__ Shared s;
    extern __shared__ ulonglong2 s_rng[];
    const int tid = threadIdx.x;
    build_move_lut(s);
    const bool queued = p.queue != nullptr;
    for (;;) {
        int g = blockIdx.x, rem = p.steps;
        if (queued) {
            if (tid == 0) s.job = queue_pop(p.queue, p.ring, p.ring_cap);
            __syncthreads();
            g = s.job;
            if (g < 0) break;
            rem = p.remaining[g];
        }
        const int n_steps = (queued && rem > p.chunk) ? p.chunk : rem;
        long long t_start = 0;
        if (queued && tid == 0) t_start = global_timer_ns();
        run_slice<OCP, 1>(p, s, s_rng, nullptr, g, n_steps, p.first != 0 && rem == p.steps);
        if (!queued) break;
        __syncthreads();  // every thread's writes of the slice precede the fence of thread 0
        if (tid == 0) {
            if (p.trace) {
                const int k = atomicAdd(p.trace_count, 1);
                if (k < p.trace_cap) {
                    unsigned sm;
                    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
                    p.trace[4 * k] = g;
                    p.trace[4 * k + 1] = t_start;
                    p.trace[4 * k + 2] = global_timer_ns();
                    p.trace[4 * k + 3] = ((long long)sm << 32) | (unsigned)n_steps;
                }
            }
            const int left = rem - n_steps;
            p.remaining[g] = left;
            __threadfence();
            if (left > 0) {
                // band of the time the tree still needs at the pace of this slice, counted down from the longest whole
                // search seen so far in this launch
                // the pace of a tree changes from slice to slice (its tree deepens, its neighbours on the SM change): half
                // the weight goes to the slices before (worth 1-2 % on the headline batch: 16.7-17.2 G playouts/s against
                // 16.6-16.8 with the last slice alone)
                float us_per_step = (float)(global_timer_ns() - t_start) * 1e-3f / (float)n_steps;
                if (rem != p.steps) us_per_step = 0.5f * us_per_step + 0.5f * p.state[g].us_per_step;
                p.state[g].us_per_step = us_per_step;
                const int whole = (int)fminf(us_per_step * (float)p.steps, 2e9f);
                const int longest = max(atomicMax(&p.queue->longest_us, whole), max(whole, 1));
                const float below = QUEUE_LEVELS_PER_OCTAVE * log2f((float)longest / fmaxf(us_per_step * (float)left, 1e-3f));
                const int level = max(0, QUEUE_LEVELS - 1 - (int)fminf(fmaxf(below, 0.f), (float)QUEUE_LEVELS));
                if (!queue_push(p.queue, p.ring, p.ring_cap, level, g)) atomicOr(&p.state[g].status, STATUS_INTERNAL);
            }
        }
    }
}

// A cluster of CLUSTER_BLOCKS blocks per tree: launches with few trees (one search), where a step of a tree is bound by what one
// SM can play.  Launched with the cluster dimension as a launch attribute; cluster c grows tree c for the whole launch.
#ifndef MCTSNC_C4_CLUSTER_BLOCKS
#define MCTSNC_C4_CLUSTER_BLOCKS 8
#endif
#ifndef MCTSNC_C4_CLUSTER_THREADS
#define MCTSNC_C4_CLUSTER_THREADS 256
#endif
constexpr int CLUSTER_BLOCKS = MCTSNC_C4_CLUSTER_BLOCKS;
constexpr int CLUSTER_THREADS = MCTSNC_C4_CLUSTER_THREADS;

template <bool OCP>
__global__ void __launch_bounds__(CLUSTER_THREADS) search_cluster_kernel(const SearchParams p) {
    __shared__ Shared s;
    extern __shared__ ulonglong2 s_rng[];
    build_move_lut(s);
    const int n_local = ((OCP ? 1 : A) * p.n_playouts) / CLUSTER_BLOCKS;   // streams this block keeps; the record cache follows
    run_slice<OCP, CLUSTER_BLOCKS>(p, s, s_rng, reinterpret_cast<int4 *>(s_rng + n_local), (int)(blockIdx.x / CLUSTER_BLOCKS), p.steps,
                                   p.first != 0);
}

}  // namespace c4
}  // namespace mctsnc
