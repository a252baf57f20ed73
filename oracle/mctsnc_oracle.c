/*
 * mctsnc_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A sequential CPU restatement of the MCTS-NC search of the reference project
 * (MarkJoson/mcts_numba_cuda).  It exists to check the CUDA library and to
 * serve as the timed CPU baseline; the product library never includes, links
 * or calls anything in this file.
 *
 * Every routine follows one numba.cuda kernel (or device function) of the
 * reference and executes it "as if all threads of a block ran in lockstep".
 * Citations are file:line inside the reference project.
 *
 *   src/mctsnc.py:1260-1290   _reset                       -> k_reset
 *   src/mctsnc.py:1293-1365   _select                      -> k_select
 *   src/mctsnc.py:1368-1681   _expand_1_{ocp,acp}_{thrifty,prodigal} -> k_expand_1
 *   src/mctsnc.py:1684-1688   _memorize_root_actions_expanded -> in mo_run
 *   src/mctsnc.py:1691-1821   _expand_2_{thrifty,prodigal} -> k_expand_2
 *   src/mctsnc.py:1824-2081   _playout_ocp / _playout_acp_* -> k_playout
 *   src/mctsnc.py:2084-2220   _backup_ocp / _backup_1_acp_* / _backup_2_acp
 *   src/mctsnc.py:2223-2375   _reduce_over_trees_* / _reduce_over_actions_*
 *   src/mctsnc.py:565-1257    the four host loops _run_<variant> -> mo_run
 *   src/mctsnc_game_mechanics.py:89-281  Connect-4 and Gomoku device functions
 *   numba/cuda/random.py (numba 0.65.0, third party, not vendored by the
 *   reference): SplitMix64 seeding, xoroshiro128+ (rotations 55/14/36), the
 *   2^64 jump, uint64 -> float32 through float64.  Restated from the published
 *   algorithm; call sites src/mctsnc.py:391-394,1435,1511,1882,1971,2061.
 *
 * Parity pin: this file reproduces, field for field, the two tree dumps the
 * reference ships (extras/mctsnc_ocp_thrifty_c4_1000steps.json and
 * extras/mctsnc_acp_thrifty_c4_1000steps.json); tests/test_oracle_golden.py
 * checks that against a digest of those files.  It also replays matches the
 * reference's authors recorded on their GPU (experiments/[...].zip of the
 * reference: step count, move, n_root, n, n_wins, playouts, depths and sizes
 * of every search) search by search, one instance per recorded player with
 * the random streams running on across searches and games;
 * tests/test_oracle_experiment_replay.py checks several hundred such searches
 * of all four variants, draws equal to 1.0f included.
 *
 * Conventions where the reference leaves behaviour undefined:
 *  - numba's uniform_float32 can return exactly 1.0f (probability 2^-25 per
 *    draw); the playout then reads legal_actions_with_count[count], a slot
 *    that holds a stale value of the same playout or was never written.  Here
 *    the per-thread legal-action array starts as zeros at every playout and is
 *    otherwise left alone, numba's negative-index wrap-around is reproduced
 *    (wrap_idx), and such draws are counted in ub_draws.
 *  - the same 1.0f draw in the OCP random-child pick indexes one past the list
 *    of expanded children; here the pick is clamped to the last child and the
 *    event is counted in ub_draws as well.
 *  - device arrays the reference leaves uninitialised (cuda.device_array) are
 *    zero here, child columns of never-expanded nodes are -1.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAX_TREE_DEPTH 2048 /* src/mctsnc.py:197 */
#define TPB_DEFAULT 512     /* MAX_THREADS_PER_BLOCK // 2, src/mctsnc.py:281 */

enum { GAME_C4 = 0, GAME_GOMOKU = 1 };
enum { OCP_THRIFTY = 0, OCP_PRODIGAL = 1, ACP_THRIFTY = 2, ACP_PRODIGAL = 3 };

typedef struct { uint64_t s0, s1; } rng_state;

#define LEGAL_LEN (512 + 1) /* src/mctsnc.py:1832 */

typedef struct {
    int8_t board[32 * 32];
    int8_t extra[4096];
    int16_t legal[LEGAL_LEN];
} playout_local;

typedef struct mo_ctx {
    int m, n, extra, A, game, T, P, variant;
    int64_t max_tree_size; /* logical limit used by expand_1 */
    int64_t cap;           /* nodes actually allocated per tree */
    float ucb_c;
    uint64_t seed;
    int64_t tree_offset;       /* global index of this context's first tree (0 unless the search is split) */
    int tpb_r, tpb_s, tpb_e1, tpb_e2, tpb_b1, tpb_b2, tpb_rot, tpb_roa;
    /* device-side arrays of the reference, src/mctsnc.py:372-404 */
    int32_t *trees;
    int32_t *trees_sizes;
    int16_t *trees_depths;
    int8_t *trees_turns;
    uint8_t *trees_leaves;
    uint8_t *trees_terminals;
    int8_t *trees_outcomes;
    int32_t *trees_ns;
    int32_t *trees_ns_wins;
    int8_t *trees_boards;
    int8_t *trees_extra_infos;
    int32_t *trees_nodes_selected;
    int32_t *trees_selected_paths;
    int16_t *trees_actions_expanded;
    int32_t *trees_playout_outcomes;
    int32_t *trees_playout_outcomes_children;
    rng_state *rng_expand_1;
    int64_t n_rng_expand_1;
    rng_state *rng_playout;
    int64_t n_rng_playout;
    int16_t *root_actions_expanded;
    int64_t *root_ns;
    uint8_t *actions_win_flags;
    int64_t *actions_ns;
    int64_t *actions_ns_wins;
    int16_t best_action;
    uint8_t best_win_flag;
    int64_t best_n, best_n_wins;
    /* bookkeeping that the reference does not have */
    int64_t steps;
    int64_t ub_draws;
    int64_t plies;
    int64_t tree_full_events;
    int32_t error;
    playout_local local; /* the per-thread local arrays of a playout, one thread at a time */
} mo_ctx;

/* ------------------------------------------------------------------------- */
/* numba.cuda.random restated                                                 */

static inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

/* init_xoroshiro128p_state: SplitMix64 of the seed, both words equal */
static void rng_seed(rng_state *s, uint64_t seed) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    s->s0 = z;
    s->s1 = z;
}

/* xoroshiro128p_next */
static inline uint64_t rng_next(rng_state *s) {
    uint64_t s0 = s->s0, s1 = s->s1;
    uint64_t result = s0 + s1;
    s1 ^= s0;
    s->s0 = rotl64(s0, 55) ^ s1 ^ (s1 << 14);
    s->s1 = rotl64(s1, 36);
    return result;
}

/* xoroshiro128p_jump: 2^64 steps ahead */
static void rng_jump(rng_state *s) {
    static const uint64_t jump[2] = {0xbeac0467eba5facbULL, 0xd86b048b86aa9922ULL};
    uint64_t s0 = 0, s1 = 0;
    for (int i = 0; i < 2; i++)
        for (int b = 0; b < 64; b++) {
            if (jump[i] & (1ULL << b)) {
                s0 ^= s->s0;
                s1 ^= s->s1;
            }
            rng_next(s);
        }
    s->s0 = s0;
    s->s1 = s1;
}

/* init_xoroshiro128p_states_cpu(states, seed, subsequence_start): state 0 is the seeded state jumped
 * subsequence_start times, state i the state i-1 jumped once more (numba/cuda/random.py:226-243) */
void mo_rng_init_states_from(rng_state *states, int64_t n, uint64_t seed, int64_t subsequence_start) {
    if (n < 1) return;
    rng_seed(&states[0], seed);
    for (int64_t i = 0; i < subsequence_start; i++) rng_jump(&states[0]);
    for (int64_t i = 1; i < n; i++) {
        states[i] = states[i - 1];
        rng_jump(&states[i]);
    }
}

void mo_rng_init_states(rng_state *states, int64_t n, uint64_t seed) { mo_rng_init_states_from(states, n, seed, 0); }

/* xoroshiro128p_uniform_float32: float32(float64(x >> 11) * 2^-53) */
static inline float rng_uniform_f32(rng_state *s) {
    uint64_t x = rng_next(s);
    double d = (double)(x >> 11) * (1.0 / 9007199254740992.0);
    return (float)d;
}

/* exposed for the tests of the generator itself */
float mo_rng_uniform_f32(rng_state *s) { return rng_uniform_f32(s); }
uint64_t mo_rng_next(rng_state *s) { return rng_next(s); }

/* ------------------------------------------------------------------------- */
/* numba array indexing: a negative index wraps once                          */

static inline int wrap_idx(mo_ctx *c, int i, int len) {
    if (i < 0) i += len;
    if (i < 0 || i >= len) { /* outside even after the wrap: no defined meaning */
        c->error |= 1;
        i = i < 0 ? 0 : len - 1;
    }
    return i;
}

static inline int8_t *bcell(mo_ctx *c, int8_t *board, int i, int j) {
    i = wrap_idx(c, i, c->m);
    j = wrap_idx(c, j, c->n);
    return &board[i * c->n + j];
}

/* ------------------------------------------------------------------------- */
/* game mechanics, src/mctsnc_game_mechanics.py                               */

/* is_action_legal_c4 :90-92, is_action_legal_gomoku :182-186 */
static int is_action_legal(mo_ctx *c, int8_t *board, int8_t *extra, int action) {
    if (c->game == GAME_C4) return extra[action] < c->m;
    return board[(action / c->n) * c->n + (action % c->n)] == 0;
}

/* take_action_c4 :95-99, take_action_gomoku :189-193 */
static void take_action(mo_ctx *c, int8_t *board, int8_t *extra, int turn, int action) {
    if (c->game == GAME_C4) {
        extra[action] += 1;
        int row = c->m - extra[action];
        *bcell(c, board, row, action) = (int8_t)turn;
    } else {
        board[(action / c->n) * c->n + (action % c->n)] = (int8_t)turn;
    }
}

/* legal_actions_playout_c4 :102-109, legal_actions_playout_gomoku :196-207 */
static void legal_actions_playout(mo_ctx *c, int8_t *board, int8_t *extra, int16_t *legal) {
    if (c->game == GAME_C4) {
        int count = 0;
        for (int j = 0; j < c->n; j++)
            if (extra[j] < c->m) legal[count++] = (int16_t)j;
        legal[LEGAL_LEN - 1] = (int16_t)count;
    } else {
        if (legal[LEGAL_LEN - 1] == 0) {
            int count = 0, k = 0;
            for (int i = 0; i < c->m; i++)
                for (int j = 0; j < c->n; j++) {
                    if (board[i * c->n + j] == 0) legal[count++] = (int16_t)k;
                    k++;
                }
            legal[LEGAL_LEN - 1] = (int16_t)count;
        }
    }
}

/* take_action_playout_c4 :112-116, take_action_playout_gomoku :210-217 */
static void take_action_playout(mo_ctx *c, int8_t *board, int8_t *extra, int turn, int action,
                                int action_ord, int16_t *legal) {
    if (c->game == GAME_C4) {
        int a = wrap_idx(c, action, c->extra);
        extra[a] += 1;
        int row = c->m - extra[a];
        *bcell(c, board, row, action) = (int8_t)turn;
    } else {
        int i = action / c->n, j = action % c->n; /* action >= 0 always holds here */
        if (action < 0) { c->error |= 2; i = 0; j = 0; }
        *bcell(c, board, i, j) = (int8_t)turn;
        int cnt = legal[LEGAL_LEN - 1];
        int16_t last = legal[wrap_idx(c, cnt - 1, LEGAL_LEN)];
        legal[wrap_idx(c, action_ord, LEGAL_LEN)] = last;
        legal[LEGAL_LEN - 1] -= 1;
    }
}

/* one direction of the line test shared by compute_outcome_c4 / _gomoku */
static int line_total(mo_ctx *c, int8_t *board, int i, int j, int di, int dj, int reach, int token) {
    int m = c->m, n = c->n, total = 0;
    for (int k = 1; k < reach; k++) {
        int ii = i + k * di, jj = j + k * dj;
        /* bounds exactly as written in the reference: only the side that can be left is tested */
        if ((di < 0 && ii < 0) || (di > 0 && ii >= m) || (dj < 0 && jj < 0) || (dj > 0 && jj >= n)) break;
        if (*bcell(c, board, ii, jj) != token) break;
        total++;
    }
    return total;
}

/* compute_outcome_c4 :119-179, compute_outcome_gomoku :220-281 */
static int compute_outcome(mo_ctx *c, int8_t *board, int8_t *extra, int turn, int last_action) {
    int last_token = -turn;
    int m = c->m, n = c->n;
    if (c->game == GAME_C4) {
        int j = last_action;
        int i = m - extra[wrap_idx(c, j, c->extra)];
        int total;
        total = line_total(c, board, i, j, -1, 0, 4, last_token) + line_total(c, board, i, j, 1, 0, 4, last_token);
        if (total >= 3) return last_token;
        total = line_total(c, board, i, j, 0, 1, 4, last_token) + line_total(c, board, i, j, 0, -1, 4, last_token);
        if (total >= 3) return last_token;
        total = line_total(c, board, i, j, -1, 1, 4, last_token) + line_total(c, board, i, j, 1, -1, 4, last_token);
        if (total >= 3) return last_token;
        total = line_total(c, board, i, j, -1, -1, 4, last_token) + line_total(c, board, i, j, 1, 1, 4, last_token);
        if (total >= 3) return last_token;
        for (int jj = 0; jj < n; jj++)
            if (extra[jj] < m) return 2;
        return 0;
    } else {
        int i = last_action / n, j = last_action % n;
        int total;
        total = line_total(c, board, i, j, -1, 0, 6, last_token) + line_total(c, board, i, j, 1, 0, 6, last_token);
        if (total == 4) return last_token;
        total = line_total(c, board, i, j, 0, 1, 6, last_token) + line_total(c, board, i, j, 0, -1, 6, last_token);
        if (total == 4) return last_token;
        total = line_total(c, board, i, j, -1, 1, 6, last_token) + line_total(c, board, i, j, 1, -1, 6, last_token);
        if (total == 4) return last_token;
        total = line_total(c, board, i, j, -1, -1, 6, last_token) + line_total(c, board, i, j, 1, 1, 6, last_token);
        if (total == 4) return last_token;
        for (int k = 0; k < m * n; k++)
            if (board[k] == 0) return 2;
        return 0;
    }
}

/* ------------------------------------------------------------------------- */
/* indexing helpers                                                           */

#define TREES(c, ti, node, col) ((c)->trees[((int64_t)(ti) * (c)->cap + (node)) * (1 + (c)->A) + (col)])
#define NODE(c, arr, ti, node) ((c)->arr[(int64_t)(ti) * (c)->cap + (node)])
#define BOARD(c, ti, node) (&(c)->trees_boards[((int64_t)(ti) * (c)->cap + (node)) * (c)->m * (c)->n])
#define EXTRA(c, ti, node) (&(c)->trees_extra_infos[((int64_t)(ti) * (c)->cap + (node)) * (c)->extra])
/* trees_actions_expanded[ti, k] with python-style negative k */
#define AE(c, ti, k) ((c)->trees_actions_expanded[(int64_t)(ti) * ((c)->A + 2) + ((k) < 0 ? (c)->A + 2 + (k) : (k))])
#define PATHS(c, ti, k) ((c)->trees_selected_paths[(int64_t)(ti) * (MAX_TREE_DEPTH + 2) + ((k) < 0 ? MAX_TREE_DEPTH + 2 + (k) : (k))])

static int pow2ceil(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

/* ------------------------------------------------------------------------- */
/* kernels                                                                    */

/* _reset, src/mctsnc.py:1260-1290 */
static void k_reset(mo_ctx *c, const int8_t *root_board, const int8_t *root_extra, int root_extra_len, int root_turn) {
    for (int ti = 0; ti < c->T; ti++) {
        TREES(c, ti, 0, 0) = -1;
        c->trees_sizes[ti] = 1;
        NODE(c, trees_depths, ti, 0) = 0;
        NODE(c, trees_turns, ti, 0) = (int8_t)root_turn;
        NODE(c, trees_leaves, ti, 0) = 1;
        NODE(c, trees_terminals, ti, 0) = 0;
        NODE(c, trees_ns, ti, 0) = 0;
        NODE(c, trees_ns_wins, ti, 0) = 0;
        memcpy(BOARD(c, ti, 0), root_board, (size_t)c->m * c->n);
        /* the reference loop lacks "e += tpb" (:1288-1290); with extra_info <= tpb_r every byte is still copied once */
        for (int e = 0; e < root_extra_len && e < c->extra; e++) EXTRA(c, ti, 0)[e] = root_extra[e];
    }
}

/* _select, src/mctsnc.py:1293-1365; the 512-wide stride-halving max/argmax is kept literally,
   because its keep-left-on-ties rule decides between equal UCBs (:1343-1351) */
static void k_select(mo_ctx *c, int ti) {
    float shared_ucbs[TPB_DEFAULT];
    int32_t shared_best_child[TPB_DEFAULT];
    int tpb = c->tpb_s;
    int A = c->A;
    int32_t node = 0;
    int depth = 0;
    PATHS(c, ti, 0) = 0;
    /* only the first pow2ceil(A) slots can hold anything but -inf */
    int width = pow2ceil(A);
    if (width > tpb) width = tpb;
    while (!NODE(c, trees_leaves, ti, node)) {
        for (int t = 0; t < width; t++) {
            if (t < A) {
                int32_t child = TREES(c, ti, node, 1 + t);
                shared_best_child[t] = child;
                if (child == -1) {
                    shared_ucbs[t] = -INFINITY;
                } else {
                    int32_t child_n = NODE(c, trees_ns, ti, child);
                    if (child_n == 0) {
                        shared_ucbs[t] = INFINITY;
                    } else {
                        /* :1337 -- numba types int32/float32 as float64, log(int32) as float64,
                           float32*float64 as float64; the float64 sum is rounded when stored to the
                           float32 shared array.  NVVM contracts the final multiply-add. */
                        double q = (double)NODE(c, trees_ns_wins, ti, child) / (double)(float)child_n;
                        double e = sqrt(log((double)NODE(c, trees_ns, ti, node)) / (double)child_n);
                        shared_ucbs[t] = (float)fma((double)c->ucb_c, e, q);
                    }
                }
            } else {
                shared_ucbs[t] = -INFINITY;
            }
        }
        /* slots width..tpb-1 are -inf and never win a strict "<" against anything, so the
           strides above `width/2` leave slots 0..width-1 untouched */
        for (int stride = width >> 1; stride > 0; stride >>= 1)
            for (int t = 0; t < stride; t++)
                if (shared_ucbs[t] < shared_ucbs[t + stride]) {
                    shared_ucbs[t] = shared_ucbs[t + stride];
                    shared_best_child[t] = shared_best_child[t + stride];
                }
        node = shared_best_child[0];
        depth++;
        PATHS(c, ti, depth) = node;
    }
    c->trees_nodes_selected[ti] = node;
    PATHS(c, ti, -1) = depth + 1;
}

/* _expand_1_* , src/mctsnc.py:1368-1681 (four variants, differences marked) */
static void k_expand_1(mo_ctx *c, int ti) {
    int A = c->A;
    uint8_t legal[512];
    int16_t shifts[512];
    int16_t map_shift_to_action[512];
    int ocp = (c->variant == OCP_THRIFTY || c->variant == OCP_PRODIGAL);
    int thrifty = (c->variant == OCP_THRIFTY || c->variant == ACP_THRIFTY);
    int32_t selected = c->trees_nodes_selected[ti];
    int8_t *board = BOARD(c, ti, selected);
    int8_t *extra = EXTRA(c, ti, selected);
    int selected_is_terminal = NODE(c, trees_terminals, ti, selected);
    for (int t = 0; t < A; t++) legal[t] = selected_is_terminal ? 0 : (uint8_t)is_action_legal(c, board, extra, t);
    int32_t size_so_far = c->trees_sizes[ti];
    int child_shift = -1;
    int pick = -3; /* rand_child_for_playout / fake_child_for_playout */
    for (int t = 0; t < A; t++) shifts[t] = -1;
    memset(map_shift_to_action, 0, sizeof(map_shift_to_action));
    if (!selected_is_terminal) {
        for (int i = 0; i < A; i++) {
            if (legal[i] && (int64_t)size_so_far + child_shift + 1 < c->max_tree_size) {
                child_shift++;
                map_shift_to_action[child_shift] = (int16_t)i;
            } else if (legal[i]) {
                c->tree_full_events++;
            }
            shifts[i] = (int16_t)child_shift;
        }
        if (child_shift >= 0) {
            AE(c, ti, -1) = (int16_t)(child_shift + 1);
            NODE(c, trees_leaves, ti, selected) = 0;
            if (ocp) {
                /* :1435/:1511 -- float32 * int64 is a float64 product, then int16() truncation */
                float u = rng_uniform_f32(&c->rng_expand_1[(int64_t)ti * c->tpb_e1]);
                int r = (int)((double)u * (double)(child_shift + 1));
                if (r > child_shift) { /* u == 1.0f: undefined in the reference, clamped here */
                    r = child_shift;
                    c->ub_draws++;
                }
                pick = thrifty ? r : map_shift_to_action[r];
            } else {
                pick = -2;
            }
        } else {
            AE(c, ti, -1) = 1;
        }
        AE(c, ti, -2) = (int16_t)pick;
    } else {
        AE(c, ti, -1) = 1;
        AE(c, ti, -2) = -1;
    }
    for (int t = 0; t < A; t++) {
        int32_t child_index = -1;
        if (legal[t]) {
            int cs = shifts[t];
            /* a legal action that did not fit (tree full) repeats the previous shift: only the action that
               first reached a shift value owns it */
            int owns = cs >= 0 && (t == 0 ? 1 : shifts[t - 1] != cs);
            if (owns) {
                child_index = size_so_far + cs;
                if (thrifty) AE(c, ti, cs) = (int16_t)t;
                else AE(c, ti, t) = (int16_t)t;
            } else if (!thrifty) {
                AE(c, ti, t) = -1;
            }
        } else if (!thrifty) {
            AE(c, ti, t) = -1;
        }
        TREES(c, ti, selected, 1 + t) = child_index;
    }
    c->trees_sizes[ti] += shifts[A - 1] + 1;
    if (!ocp && (selected_is_terminal || pick == -3)) AE(c, ti, 0) = 0; /* :1603-1604, :1680-1681 */
}

/* _expand_2_thrifty / _expand_2_prodigal, src/mctsnc.py:1691-1821, one (tree, action) block */
static void k_expand_2(mo_ctx *c, int ti, int action) {
    if (action < 0) return;
    int mode = AE(c, ti, -2);
    int thrifty = (c->variant == OCP_THRIFTY || c->variant == ACP_THRIFTY);
    if (!thrifty && (mode == -1 || mode == -3)) return;
    int32_t selected = c->trees_nodes_selected[ti];
    if (NODE(c, trees_terminals, ti, selected)) return;
    int32_t child = TREES(c, ti, selected, 1 + action);
    if (child < 0) return; /* thrifty, tree full: the fake entry; the reference would index child -1 here */
    int8_t *cb = BOARD(c, ti, child);
    int8_t *ce = EXTRA(c, ti, child);
    memcpy(cb, BOARD(c, ti, selected), (size_t)c->m * c->n);
    memcpy(ce, EXTRA(c, ti, selected), (size_t)c->extra);
    int turn = NODE(c, trees_turns, ti, selected);
    take_action(c, cb, ce, turn, action);
    TREES(c, ti, child, 0) = selected;
    NODE(c, trees_turns, ti, child) = (int8_t)(-turn);
    NODE(c, trees_leaves, ti, child) = 1;
    int outcome = compute_outcome(c, cb, ce, -turn, action);
    NODE(c, trees_terminals, ti, child) = (outcome == -1 || outcome == 0 || outcome == 1);
    NODE(c, trees_outcomes, ti, child) = (int8_t)outcome;
    NODE(c, trees_ns, ti, child) = 0;
    NODE(c, trees_ns_wins, ti, child) = 0;
    NODE(c, trees_depths, ti, child) = (int16_t)(NODE(c, trees_depths, ti, selected) + 1);
}

/* the per-thread body of the three playout kernels, src/mctsnc.py:1870-1890 (same text at :1959-1979, :2049-2069);
   returns the outcome in {-1,0,1} */
static int playout_thread(mo_ctx *c, playout_local *L, int ti, int32_t node, int last_action, rng_state *rs) {
    memcpy(L->board, BOARD(c, ti, node), (size_t)c->m * c->n);
    memcpy(L->extra, EXTRA(c, ti, node), (size_t)c->extra);
    memset(L->legal, 0, sizeof(L->legal)); /* convention: a fresh local array reads as zeros */
    int turn = NODE(c, trees_turns, ti, node);
    int outcome = last_action != -1 ? compute_outcome(c, L->board, L->extra, turn, last_action) : 2;
    for (int guard = 0;; guard++) {
        if (outcome == -1 || outcome == 0 || outcome == 1) return outcome;
        if (guard >= 4096) { /* only reachable after a 1.0f draw has put list and board out of step (the reference
                                would loop on); the CUDA replay gives up at the same point with the same answer */
            c->error |= 16;
            return 0;
        }
        legal_actions_playout(c, L->board, L->extra, L->legal);
        int count = L->legal[LEGAL_LEN - 1];
        /* :1882 -- float32 * int16 is a float32 product, then int16() truncation */
        float u = rng_uniform_f32(rs);
        float prod = u * (float)count;
        int action_ord = (int)(int16_t)(int)prod;
        if (u >= 1.0f) c->ub_draws++;
        last_action = L->legal[wrap_idx(c, action_ord, LEGAL_LEN)];
        take_action_playout(c, L->board, L->extra, turn, last_action, action_ord, L->legal);
        turn = -turn;
        c->plies++;
        outcome = compute_outcome(c, L->board, L->extra, turn, last_action);
    }
}

/* _playout_ocp, src/mctsnc.py:1824-1902 */
static void k_playout_ocp(mo_ctx *c, int ti) {
    playout_local *L = &c->local;
    int32_t node = c->trees_nodes_selected[ti];
    int pick = AE(c, ti, -2);
    int last_action = -1;
    if (pick >= 0) {
        last_action = AE(c, ti, pick);
        node = TREES(c, ti, node, 1 + last_action);
    }
    int32_t neg = 0, pos = 0;
    if (NODE(c, trees_terminals, ti, node)) {
        int o = NODE(c, trees_outcomes, ti, node);
        neg = o == -1 ? c->P : 0;
        pos = o == 1 ? c->P : 0;
    } else {
        for (int t = 0; t < c->P; t++) {
            int o = playout_thread(c, L, ti, node, last_action, &c->rng_playout[(int64_t)ti * c->P + t]);
            if (o == -1) neg++;
            else if (o == 1) pos++;
        }
    }
    c->trees_playout_outcomes[ti * 2 + 0] = neg;
    c->trees_playout_outcomes[ti * 2 + 1] = pos;
}

/* _playout_acp_thrifty / _playout_acp_prodigal, src/mctsnc.py:1905-2081, one (tree, action) block */
static void k_playout_acp(mo_ctx *c, int ti, int action) {
    playout_local *L = &c->local;
    if (action < 0) return;
    int32_t node = c->trees_nodes_selected[ti];
    int mode = AE(c, ti, -2);
    int last_action = -1;
    if (mode == -2) {
        last_action = action;
        node = TREES(c, ti, node, 1 + last_action);
    }
    int32_t neg = 0, pos = 0;
    if (NODE(c, trees_terminals, ti, node)) {
        int o = NODE(c, trees_outcomes, ti, node);
        neg = o == -1 ? c->P : 0;
        pos = o == 1 ? c->P : 0;
        if (mode != -2) { /* terminal node was the selected one */
            c->trees_playout_outcomes[ti * 2 + 0] = neg;
            c->trees_playout_outcomes[ti * 2 + 1] = pos;
            return;
        }
    } else {
        for (int t = 0; t < c->P; t++) {
            /* :1938 / :2028 */
            int64_t t_global = (int64_t)ti * c->A * c->P + (int64_t)action * c->P + t;
            int o = playout_thread(c, L, ti, node, last_action, &c->rng_playout[t_global]);
            if (o == -1) neg++;
            else if (o == 1) pos++;
        }
    }
    c->trees_playout_outcomes_children[(ti * c->A + action) * 2 + 0] = neg;
    c->trees_playout_outcomes_children[(ti * c->A + action) * 2 + 1] = pos;
}

static void credit(mo_ctx *c, int ti, int32_t node, int64_t n, int32_t neg, int32_t pos) {
    NODE(c, trees_ns, ti, node) += (int32_t)n;
    if (NODE(c, trees_turns, ti, node) == 1) NODE(c, trees_ns_wins, ti, node) += neg;
    else NODE(c, trees_ns_wins, ti, node) += pos;
}

/* _backup_ocp, src/mctsnc.py:2084-2114 */
static void k_backup_ocp(mo_ctx *c, int ti) {
    int32_t neg = c->trees_playout_outcomes[ti * 2 + 0], pos = c->trees_playout_outcomes[ti * 2 + 1];
    int path_length = PATHS(c, ti, -1);
    for (int e = 0; e < path_length; e++) credit(c, ti, PATHS(c, ti, e), c->P, neg, pos);
    int32_t node = c->trees_nodes_selected[ti];
    int pick = AE(c, ti, -2);
    if (pick != -1 && pick != -3) { /* the reference lets -3 through and indexes with it (:2107-2108); not followed */
        int last_action = AE(c, ti, pick);
        node = TREES(c, ti, node, 1 + last_action);
        credit(c, ti, node, c->P, neg, pos);
    }
}

/* _backup_1_acp_thrifty / _backup_1_acp_prodigal, src/mctsnc.py:2117-2194 */
static void k_backup_1_acp(mo_ctx *c, int ti) {
    if (AE(c, ti, -2) != -2) return;
    int thrifty = c->variant == ACP_THRIFTY;
    int32_t selected = c->trees_nodes_selected[ti];
    int32_t neg_sum = 0, pos_sum = 0;
    int limit = thrifty ? AE(c, ti, -1) : c->A;
    for (int t = 0; t < limit; t++) {
        int a;
        if (thrifty) a = AE(c, ti, t);
        else {
            if (AE(c, ti, t) == -1) continue;
            a = t;
        }
        int32_t neg = c->trees_playout_outcomes_children[(ti * c->A + a) * 2 + 0];
        int32_t pos = c->trees_playout_outcomes_children[(ti * c->A + a) * 2 + 1];
        credit(c, ti, TREES(c, ti, selected, 1 + a), c->P, neg, pos);
        neg_sum += neg;
        pos_sum += pos;
    }
    c->trees_playout_outcomes[ti * 2 + 0] = neg_sum;
    c->trees_playout_outcomes[ti * 2 + 1] = pos_sum;
}

/* _backup_2_acp, src/mctsnc.py:2197-2220 */
static void k_backup_2_acp(mo_ctx *c, int ti) {
    int32_t neg = c->trees_playout_outcomes[ti * 2 + 0], pos = c->trees_playout_outcomes[ti * 2 + 1];
    int n_expanded = AE(c, ti, -1);
    if (n_expanded == 0) n_expanded = 1;
    int64_t total = (int64_t)c->P * n_expanded;
    int path_length = PATHS(c, ti, -1);
    for (int e = 0; e < path_length; e++) credit(c, ti, PATHS(c, ti, e), total, neg, pos);
}

/* _reduce_over_trees_{thrifty,prodigal} :2223-2296 and _reduce_over_actions_{thrifty,prodigal} :2299-2375 */
static void k_reduce(mo_ctx *c, int root_turn) {
    int A = c->A;
    int thrifty = (c->variant == OCP_THRIFTY || c->variant == ACP_THRIFTY);
    int n_root_actions = c->root_actions_expanded[A + 1];
    int n_blocks = thrifty ? n_root_actions : A;
    memset(c->root_ns, 0, sizeof(int64_t) * A);
    memset(c->actions_ns, 0, sizeof(int64_t) * A);
    memset(c->actions_ns_wins, 0, sizeof(int64_t) * A);
    memset(c->actions_win_flags, 0, A);
    for (int b = 0; b < n_blocks; b++) {
        int action = thrifty ? c->root_actions_expanded[b] : b;
        int64_t s_root = 0, s_n = 0, s_w = 0;
        if (thrifty || c->root_actions_expanded[action] != -1) {
            for (int t = 0; t < c->T; t++) {
                s_root += NODE(c, trees_ns, t, 0);
                int32_t an = TREES(c, t, 0, 1 + action);
                s_n += NODE(c, trees_ns, t, an);
                s_w += NODE(c, trees_ns_wins, t, an);
            }
        }
        c->root_ns[b] = s_root;
        c->actions_ns[b] = s_n;
        c->actions_ns_wins[b] = s_w;
        int32_t an0 = TREES(c, 0, 0, 1 + action);
        c->actions_win_flags[b] = an0 != -1 && NODE(c, trees_terminals, 0, an0) && NODE(c, trees_outcomes, 0, an0) == root_turn;
    }
    /* lexicographic max/argmax over (win_flag, n, n_wins), stride-halving, left kept on ties */
    int tpb = c->tpb_roa;
    int16_t s_a[512];
    uint8_t s_f[512];
    int64_t s_n[512], s_w[512];
    int limit = thrifty ? n_root_actions : A;
    for (int a = 0; a < tpb; a++) {
        s_a[a] = (int16_t)a;
        if (a < limit) {
            s_f[a] = c->actions_win_flags[a];
            s_n[a] = c->actions_ns[a];
            s_w[a] = c->actions_ns_wins[a];
        } else {
            s_f[a] = 0;
            s_n[a] = 0;
            s_w[a] = 0;
        }
    }
    for (int stride = tpb >> 1; stride > 0; stride >>= 1)
        for (int a = 0; a < stride; a++) {
            int b = a + stride;
            if ((s_f[a] < s_f[b]) || (s_f[a] == s_f[b] && s_n[a] < s_n[b]) ||
                (s_f[a] == s_f[b] && s_n[a] == s_n[b] && s_w[a] < s_w[b])) {
                s_a[a] = s_a[b];
                s_n[a] = s_n[b];
                s_w[a] = s_w[b];
                s_f[a] = s_f[b];
            }
        }
    c->best_action = s_a[0];
    c->best_win_flag = s_f[0];
    c->best_n = s_n[0];
    c->best_n_wins = s_w[0];
    if (thrifty) c->best_action = c->root_actions_expanded[c->best_action]; /* :722, :1069 */
}

/* ------------------------------------------------------------------------- */
/* public API                                                                 */

mo_ctx *mo_create(int m, int n, int extra, int A, int game, int T, int P, int variant, int64_t max_tree_size,
                  int64_t cap, float ucb_c, uint64_t seed) {
    mo_ctx *c = (mo_ctx *)calloc(1, sizeof(mo_ctx));
    if (!c) return NULL;
    c->m = m; c->n = n; c->extra = extra < 1 ? 1 : extra; c->A = A; c->game = game; c->T = T; c->P = P;
    c->variant = variant; c->max_tree_size = max_tree_size; c->cap = cap < max_tree_size ? cap : max_tree_size;
    c->ucb_c = ucb_c; c->seed = seed;
    /* tpb table, src/mctsnc.py:360-370 */
    int tpb_board = pow2ceil(m * n), tpb_extra = pow2ceil(c->extra), tpb_actions = pow2ceil(A);
    int mx = tpb_board > tpb_extra ? tpb_board : tpb_extra;
    c->tpb_r = mx < TPB_DEFAULT ? mx : TPB_DEFAULT;
    c->tpb_s = TPB_DEFAULT;
    mx = c->tpb_r > tpb_actions ? c->tpb_r : tpb_actions;
    c->tpb_e1 = mx < TPB_DEFAULT ? mx : TPB_DEFAULT;
    c->tpb_e2 = c->tpb_r;
    c->tpb_b1 = tpb_actions;
    c->tpb_b2 = TPB_DEFAULT;
    c->tpb_rot = pow2ceil(T);
    c->tpb_roa = tpb_actions;
    int64_t S = c->cap;
    size_t TS = (size_t)T * S;
    c->trees = (int32_t *)malloc(TS * (1 + A) * sizeof(int32_t));
    if (c->trees) memset(c->trees, 0xFF, TS * (1 + A) * sizeof(int32_t));
    c->trees_sizes = (int32_t *)calloc(T, sizeof(int32_t));
    c->trees_depths = (int16_t *)calloc(TS, sizeof(int16_t));
    c->trees_turns = (int8_t *)calloc(TS, 1);
    c->trees_leaves = (uint8_t *)calloc(TS, 1);
    c->trees_terminals = (uint8_t *)calloc(TS, 1);
    c->trees_outcomes = (int8_t *)calloc(TS, 1);
    c->trees_ns = (int32_t *)calloc(TS, sizeof(int32_t));
    c->trees_ns_wins = (int32_t *)calloc(TS, sizeof(int32_t));
    c->trees_boards = (int8_t *)calloc(TS * m * n, 1);
    c->trees_extra_infos = (int8_t *)calloc(TS * c->extra, 1);
    c->trees_nodes_selected = (int32_t *)calloc(T, sizeof(int32_t));
    c->trees_selected_paths = (int32_t *)calloc((size_t)T * (MAX_TREE_DEPTH + 2), sizeof(int32_t));
    c->trees_actions_expanded = (int16_t *)calloc((size_t)T * (A + 2), sizeof(int16_t));
    c->trees_playout_outcomes = (int32_t *)calloc((size_t)T * 2, sizeof(int32_t));
    c->trees_playout_outcomes_children = (int32_t *)calloc((size_t)T * A * 2, sizeof(int32_t));
    c->root_actions_expanded = (int16_t *)calloc(A + 2, sizeof(int16_t));
    c->root_ns = (int64_t *)calloc(A, sizeof(int64_t));
    c->actions_win_flags = (uint8_t *)calloc(A, 1);
    c->actions_ns = (int64_t *)calloc(A, sizeof(int64_t));
    c->actions_ns_wins = (int64_t *)calloc(A, sizeof(int64_t));
    /* src/mctsnc.py:390-394 */
    if (variant == OCP_THRIFTY || variant == OCP_PRODIGAL) {
        c->n_rng_expand_1 = (int64_t)T * c->tpb_e1;
        c->n_rng_playout = (int64_t)T * P;
    } else {
        c->n_rng_expand_1 = 0;
        c->n_rng_playout = (int64_t)T * A * P;
    }
    c->rng_expand_1 = (rng_state *)calloc(c->n_rng_expand_1 > 0 ? c->n_rng_expand_1 : 1, sizeof(rng_state));
    c->rng_playout = (rng_state *)calloc(c->n_rng_playout, sizeof(rng_state));
    if (!c->trees || !c->trees_boards || !c->rng_playout) { c->error |= 4; return c; }
    mo_rng_init_states(c->rng_expand_1, c->n_rng_expand_1, seed);
    mo_rng_init_states(c->rng_playout, c->n_rng_playout, seed);
    return c;
}

/* init_device_side_arrays() re-creates the generators, src/mctsnc.py:390-394.  With a tree offset the context grows the
 * trees [offset, offset + T) of a larger search: tree t of the context draws from the streams tree offset + t has in the
 * reference's arrays (stream index tree * A * P + action * P + thread, :1938, :2028; OCP: tree * P + thread and
 * tree * tpb_e1), which is how a search is split over several devices without changing its result. */
void mo_reset_rng(mo_ctx *c) {
    int64_t per_tree = c->n_rng_playout / c->T;
    mo_rng_init_states_from(c->rng_expand_1, c->n_rng_expand_1, c->seed, c->tree_offset * (int64_t)c->tpb_e1);
    mo_rng_init_states_from(c->rng_playout, c->n_rng_playout, c->seed, c->tree_offset * per_tree);
}

void mo_set_tree_offset(mo_ctx *c, int64_t tree_offset) {
    c->tree_offset = tree_offset;
    mo_reset_rng(c);
}

void mo_destroy(mo_ctx *c) {
    if (!c) return;
    free(c->trees); free(c->trees_sizes); free(c->trees_depths); free(c->trees_turns); free(c->trees_leaves);
    free(c->trees_terminals); free(c->trees_outcomes); free(c->trees_ns); free(c->trees_ns_wins);
    free(c->trees_boards); free(c->trees_extra_infos); free(c->trees_nodes_selected); free(c->trees_selected_paths);
    free(c->trees_actions_expanded); free(c->trees_playout_outcomes); free(c->trees_playout_outcomes_children);
    free(c->rng_expand_1); free(c->rng_playout); free(c->root_actions_expanded); free(c->root_ns);
    free(c->actions_win_flags); free(c->actions_ns); free(c->actions_ns_wins);
    free(c);
}

/* the host loop, src/mctsnc.py:565-1257; `trace`, if not NULL, receives 4 int32 per (step, tree):
   selected node, number of expanded actions, -1 wins, +1 wins of the step */
int mo_run(mo_ctx *c, const int8_t *root_board, const int8_t *root_extra, int root_extra_len, int root_turn,
           int64_t steps, int32_t *trace) {
    int A = c->A, T = c->T;
    int ocp = (c->variant == OCP_THRIFTY || c->variant == OCP_PRODIGAL);
    int thrifty = (c->variant == OCP_THRIFTY || c->variant == ACP_THRIFTY);
    int8_t zero = 0;
    if (!root_extra) { root_extra = &zero; root_extra_len = 1; }
    k_reset(c, root_board, root_extra, root_extra_len, root_turn);
    c->steps = 0;
    c->plies = 0;      /* the bookkeeping counters describe one search */
    c->ub_draws = 0;
    c->tree_full_events = 0;
    for (int64_t step = 0; step < steps; step++) {
        for (int ti = 0; ti < T; ti++) {
            if ((int64_t)c->trees_sizes[ti] + A > c->cap && c->cap < c->max_tree_size) { c->error |= 8; return c->error; }
            k_select(c, ti);
        }
        for (int ti = 0; ti < T; ti++) k_expand_1(c, ti);
        if (step == 0) memcpy(c->root_actions_expanded, &AE(c, 0, 0), sizeof(int16_t) * (A + 2));
        for (int ti = 0; ti < T; ti++) {
            if (thrifty) {
                int cnt = AE(c, ti, -1); /* _flatten_trees_actions_expanded_thrifty :436-446 */
                for (int k = 0; k < cnt; k++) k_expand_2(c, ti, AE(c, ti, k));
            } else {
                for (int a = 0; a < A; a++)
                    if (AE(c, ti, a) >= 0) k_expand_2(c, ti, a);
            }
        }
        for (int ti = 0; ti < T; ti++) {
            if (ocp) {
                k_playout_ocp(c, ti);
            } else if (thrifty) {
                int cnt = AE(c, ti, -1);
                for (int k = 0; k < cnt; k++) k_playout_acp(c, ti, AE(c, ti, k));
            } else {
                for (int a = 0; a < A; a++)
                    if (AE(c, ti, a) >= 0) k_playout_acp(c, ti, a);
            }
        }
        for (int ti = 0; ti < T; ti++) {
            if (ocp) k_backup_ocp(c, ti);
            else {
                k_backup_1_acp(c, ti);
                k_backup_2_acp(c, ti);
            }
            if (trace) {
                int32_t *tr = trace + (step * T + ti) * 4;
                tr[0] = c->trees_nodes_selected[ti];
                tr[1] = AE(c, ti, -1);
                tr[2] = c->trees_playout_outcomes[ti * 2 + 0];
                tr[3] = c->trees_playout_outcomes[ti * 2 + 1];
            }
        }
        c->steps++;
    }
    k_reduce(c, root_turn);
    return c->error;
}

/* field access for the ctypes wrapper */
enum {
    F_TREES = 0, F_SIZES, F_DEPTHS, F_TURNS, F_LEAVES, F_TERMINALS, F_OUTCOMES, F_NS, F_NS_WINS, F_BOARDS,
    F_EXTRA_INFOS, F_NODES_SELECTED, F_SELECTED_PATHS, F_ACTIONS_EXPANDED, F_PLAYOUT_OUTCOMES,
    F_PLAYOUT_OUTCOMES_CHILDREN, F_ROOT_ACTIONS_EXPANDED, F_ROOT_NS, F_ACTIONS_WIN_FLAGS, F_ACTIONS_NS,
    F_ACTIONS_NS_WINS, F_RNG_EXPAND_1, F_RNG_PLAYOUT
};

void *mo_field(mo_ctx *c, int f) {
    switch (f) {
    case F_TREES: return c->trees;
    case F_SIZES: return c->trees_sizes;
    case F_DEPTHS: return c->trees_depths;
    case F_TURNS: return c->trees_turns;
    case F_LEAVES: return c->trees_leaves;
    case F_TERMINALS: return c->trees_terminals;
    case F_OUTCOMES: return c->trees_outcomes;
    case F_NS: return c->trees_ns;
    case F_NS_WINS: return c->trees_ns_wins;
    case F_BOARDS: return c->trees_boards;
    case F_EXTRA_INFOS: return c->trees_extra_infos;
    case F_NODES_SELECTED: return c->trees_nodes_selected;
    case F_SELECTED_PATHS: return c->trees_selected_paths;
    case F_ACTIONS_EXPANDED: return c->trees_actions_expanded;
    case F_PLAYOUT_OUTCOMES: return c->trees_playout_outcomes;
    case F_PLAYOUT_OUTCOMES_CHILDREN: return c->trees_playout_outcomes_children;
    case F_ROOT_ACTIONS_EXPANDED: return c->root_actions_expanded;
    case F_ROOT_NS: return c->root_ns;
    case F_ACTIONS_WIN_FLAGS: return c->actions_win_flags;
    case F_ACTIONS_NS: return c->actions_ns;
    case F_ACTIONS_NS_WINS: return c->actions_ns_wins;
    case F_RNG_EXPAND_1: return c->rng_expand_1;
    case F_RNG_PLAYOUT: return c->rng_playout;
    }
    return NULL;
}

int64_t mo_cap(mo_ctx *c) { return c->cap; }
int64_t mo_steps(mo_ctx *c) { return c->steps; }
int64_t mo_ub_draws(mo_ctx *c) { return c->ub_draws; }
int64_t mo_plies(mo_ctx *c) { return c->plies; }
int64_t mo_tree_full_events(mo_ctx *c) { return c->tree_full_events; }
int mo_error(mo_ctx *c) { return c->error; }
int mo_best_action(mo_ctx *c) { return c->best_action; }
int mo_best_win_flag(mo_ctx *c) { return c->best_win_flag; }
int64_t mo_best_n(mo_ctx *c) { return c->best_n; }
int64_t mo_best_n_wins(mo_ctx *c) { return c->best_n_wins; }
int mo_tpb_e1(mo_ctx *c) { return c->tpb_e1; }

/* ------------------------------------------------------------------------- */
/* game mechanics alone, for the tests that pin them to the reference's CPU classes (src/c4.py, src/gomoku.py):
   plays `n_actions` actions from the empty board with take_action, first player +1 (src/mcts.py:63), and writes the
   value of compute_outcome after every action (2 = game ongoing) */
int mo_replay_game(int game, int m, int n, const int16_t *actions, int n_actions, int8_t *outcomes, int8_t *final_board) {
    mo_ctx c;
    memset(&c, 0, sizeof(c));
    c.game = game; c.m = m; c.n = n; c.extra = game == GAME_C4 ? n : 1; c.A = game == GAME_C4 ? n : m * n;
    int8_t board[32 * 32];
    int8_t extra[64];
    memset(board, 0, sizeof(board));
    memset(extra, 0, sizeof(extra));
    int turn = 1;
    for (int k = 0; k < n_actions; k++) {
        if (!is_action_legal(&c, board, extra, actions[k])) return -(k + 1);
        take_action(&c, board, extra, turn, actions[k]);
        turn = -turn;
        outcomes[k] = (int8_t)compute_outcome(&c, board, extra, turn, actions[k]);
    }
    memcpy(final_board, board, (size_t)m * n);
    return c.error;
}
