/*
 * mctsnc_b200.h -- C ABI of libmctsnc_b200.so, the sm_100a implementation of the MCTS-NC search hot path.
 *
 * Plain C types only (no CUDA, no torch types).  Every function returns 0 on success, a positive cudaError_t value
 * when the CUDA runtime failed, or one of the negative MCTSNC_E_* codes; mctsnc_error_string() turns any of them
 * into text.  A handle is not thread-safe; different handles may be used from different threads.
 *
 * Each entry point names the part of the reference (MarkJoson/mcts_numba_cuda, paths inside that project) that it
 * replaces.  Where the reference launches 4-6 numba.cuda kernels per search step from a Python loop, this library
 * runs the whole loop of a search (or of a batch of independent searches) on the device.
 */
#ifndef MCTSNC_B200_H
#define MCTSNC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* games: the reference switches between them by editing src/mctsnc_game_mechanics.py:59-87 */
#define MCTSNC_GAME_C4 0     /* src/mctsnc_game_mechanics.py:89-179  */
#define MCTSNC_GAME_GOMOKU 1 /* src/mctsnc_game_mechanics.py:181-281 */

/* MCTSNC.VARIANTS, src/mctsnc.py:180 (same order) */
#define MCTSNC_OCP_THRIFTY 0
#define MCTSNC_OCP_PRODIGAL 1
#define MCTSNC_ACP_THRIFTY 2
#define MCTSNC_ACP_PRODIGAL 3

/* library error codes (CUDA runtime errors are passed through as positive numbers) */
#define MCTSNC_E_BAD_ARGUMENT -1
#define MCTSNC_E_UNSUPPORTED -2
#define MCTSNC_E_NO_MEMORY -3
#define MCTSNC_E_BAD_ROOT -4      /* board and extra_info of a root do not describe a reachable position */
#define MCTSNC_E_CAPACITY -5      /* batch larger than max_batch, or steps beyond the node capacity of a time-less run */
#define MCTSNC_E_NO_DEVICE -6

/* bits of mctsnc_result.status */
#define MCTSNC_STATUS_TREE_FULL 1u   /* some tree reached max_tree_size; the reference's behaviour there is not followed */
#define MCTSNC_STATUS_UB_DRAW 2u     /* a uniform draw was exactly 1.0f (see ub_draws) */
#define MCTSNC_STATUS_INTERNAL 4u    /* an index check inside a kernel failed; results are not to be trusted */

typedef struct mctsnc_handle mctsnc_handle;

/* Constructor arguments of MCTSNC (src/mctsnc.py:199-204) plus what init_device_side_arrays() derives (:318-407). */
typedef struct mctsnc_config {
    int32_t board_rows;         /* state_board_shape[0] */
    int32_t board_cols;         /* state_board_shape[1] */
    int32_t extra_info_memory;  /* state_extra_info_memory (bytes) */
    int32_t max_actions;        /* state_max_actions */
    int32_t game;               /* MCTSNC_GAME_* */
    int32_t variant;            /* MCTSNC_OCP_THRIFTY .. MCTSNC_ACP_PRODIGAL */
    int32_t n_trees;            /* trees grown by THIS handle for every search */
    int32_t n_playouts;         /* power of two, <= 512 */
    float ucb_c;
    int32_t device;             /* CUDA device ordinal */
    uint64_t seed;
    int64_t max_tree_size;      /* the reference's node limit per tree (src/mctsnc.py:357-358) */
    int64_t node_capacity;      /* nodes to allocate per tree, <= max_tree_size; a search of s steps needs s*max_actions+1 */
    int32_t max_batch;          /* independent searches that one mctsnc_run_batch call may hold */
    /* root-parallel sharding over several handles (one per GPU): this handle grows the trees
       [tree_offset, tree_offset + n_trees) of a search with n_trees_global trees in total; a single-GPU
       search has tree_offset = 0 and n_trees_global = n_trees.  The random streams are those of the
       single-GPU search with n_trees_global trees (src/mctsnc.py:390-394, :1938, :2028). */
    int32_t tree_offset;
    int32_t n_trees_global;
    int32_t threads_per_tree;   /* 0 = let the library choose (Connect-4 launches with few trees and more than 256 games
                                   a step then grow every tree with a cluster of 8 blocks; the environment
                                   variable MCTSNC_B200_NO_CLUSTER=1, read at mctsnc_create, keeps one block per tree);
                                   else threads of the one block that grows a tree */
    int32_t reserved;
} mctsnc_config;

/* What run() leaves behind in the reference: best_* (src/mctsnc.py:1242-1246) and the per-action arrays behind
   actions_info (:531-563).  Per-action arrays are indexed by ACTION for every variant (the thrifty variants of the
   reference index them by ordinal among the root's expanded actions; root_actions_expanded gives that order). */
#define MCTSNC_MAX_ACTIONS 512
typedef struct mctsnc_result {
    int32_t best_action;
    int32_t best_win_flag;
    int64_t best_n;
    int64_t best_n_wins;
    int64_t steps;               /* search steps carried out */
    int64_t playouts;            /* sum over this handle's trees of the root visit count */
    int64_t plies;               /* moves played inside playouts (device counter) */
    int64_t ub_draws;            /* draws equal to 1.0f met inside playouts or the OCP child pick */
    uint32_t status;             /* MCTSNC_STATUS_* bits */
    int32_t n_root_actions;      /* actions expanded at the root (tree 0) */
    float device_ms;             /* CUDA-event time of the search kernels of the call this result came from */
    int32_t max_depth;
    int64_t total_nodes;         /* sum of tree sizes */
    int64_t depth_sum;           /* sum of node depths over all nodes (for mean_depth) */
    int32_t max_size;
    int32_t reserved;
    /* time spent in the four stages of the steps (select, expand, playouts, backup), milliseconds, mean over this
       handle's trees of the time their blocks spent there (SM cycle counter at the nominal clock); the reference's
       time_select / time_expand / time_playout / time_backup (src/mctsnc.py:606-686) are host clocks around launches */
    float stage_ms[4];
    float reduce_ms[2];          /* CUDA-event time of the two final reductions (mctsnc_run only; 0 for batch calls) */
    int64_t root_ns[MCTSNC_MAX_ACTIONS];         /* sum over trees of the root visit count, 0 for actions not expanded */
    int64_t actions_ns[MCTSNC_MAX_ACTIONS];
    int64_t actions_ns_wins[MCTSNC_MAX_ACTIONS];
    uint8_t actions_win_flags[MCTSNC_MAX_ACTIONS];
    uint8_t actions_expanded[MCTSNC_MAX_ACTIONS]; /* 1 if the action was expanded at the root of tree 0 */
} mctsnc_result;

/* Replaces MCTSNC.__init__ + init_device_side_arrays (src/mctsnc.py:199-276, :318-407): validates, allocates the
   tree pools and creates the random streams (numba create_xoroshiro128p_states, called at :390-394). */
int mctsnc_create(const mctsnc_config *cfg, mctsnc_handle **out);
int mctsnc_destroy(mctsnc_handle *h);

/* Re-creates the random streams from the seed, as a fresh init_device_side_arrays() does (src/mctsnc.py:390-394).
   Streams otherwise continue across searches, as in the reference. */
int mctsnc_reset_rng(mctsnc_handle *h);

/* Replaces MCTSNC.run -> _run_<variant> (src/mctsnc.py:409-434, :565-1257): one search from one root.
   board: int8[rows*cols] row-major in {-1,0,1}; extra_info: int8[extra_info_memory] or NULL; turn in {-1,+1}.
   Budget as in :597-601: stops when steps_limit steps are done or time_limit_s has passed (either may be "none":
   steps_limit < 0, time_limit_s <= 0); the clock is read between launches of `steps_per_launch` steps. */
int mctsnc_run(mctsnc_handle *h, const int8_t *board, const int8_t *extra_info, int32_t turn, int64_t steps_limit,
               double time_limit_s, mctsnc_result *out);

/* `batch` independent searches (same configuration, different roots) in one launch: the throughput form of run().
   boards: int8[batch][rows*cols]; extra_infos: int8[batch][extra_info_memory] or NULL; turns: int8[batch];
   results: mctsnc_result[batch].  Every search draws from its own copy of the streams; with reseed != 0 each copy is
   first re-created from the seed, so that search i equals a fresh single run() on root i.  Host buffers. */
int mctsnc_run_batch(mctsnc_handle *h, int32_t batch, const int8_t *boards, const int8_t *extra_infos,
                     const int8_t *turns, int64_t steps, int32_t reseed, mctsnc_result *results);

/* The two halves of run_batch for callers that keep data on the device and add their own exchange step
   (multi-GPU root parallelism): search writes, per search, 3*max_actions int64 partial sums
   [root_ns | actions_ns | actions_ns_wins] (what _reduce_over_trees_* computes, src/mctsnc.py:2223-2296) into the
   DEVICE buffer partial_sums; after the caller has summed those buffers over the handles of a search (all-reduce),
   finish runs the argmax of _reduce_over_actions_* (src/mctsnc.py:2299-2375) on the summed values and fills results.
   stream: a cudaStream_t (NULL = default stream).  search is asynchronous.  boards_host == NULL searches the roots of
   the previous call again (they stay resident on the device).  One search per handle may be in flight: a call that
   stages new roots first waits until the previous call's copies have read the (single) pinned staging buffer, and the
   timing events behind device_ms are those of the last search call.  finish synchronises and copies the results to the
   host, unless results == NULL: then it only launches the argmax kernel and returns. */
int mctsnc_search_batch_device(mctsnc_handle *h, int32_t batch, const int8_t *boards_host, const int8_t *extra_infos_host,
                               const int8_t *turns_host, int64_t steps, int32_t reseed, int64_t *partial_sums_device,
                               void *stream);
int mctsnc_finish_batch_device(mctsnc_handle *h, int32_t batch, const int64_t *summed_device, mctsnc_result *results,
                               void *stream);

/* mctsnc_search_batch_device in its two parts, for callers that overlap the exchange of one batch with the search of the
   next: launch stages the roots (or reuses the resident ones), re-seeds and runs the searches; reduce_trees forms the
   partial sums (_reduce_over_trees_*, src/mctsnc.py:2223-2296).  reduce_trees and finish share per-handle buffers (win
   flags, statistics): the caller orders reduce_trees of a batch after the finish of the batch before (an event), the
   searches themselves need no such wait. */
int mctsnc_launch_batch_device(mctsnc_handle *h, int32_t batch, const int8_t *boards_host, const int8_t *extra_infos_host,
                               const int8_t *turns_host, int64_t steps, int32_t reseed, void *stream);
int mctsnc_reduce_trees_device(mctsnc_handle *h, int32_t batch, int64_t *partial_sums_device, void *stream);

/* Replaces the copy_to_host calls of _json_dump (src/mctsnc.py:2393-2438): converts the trees of search `search`
   (0 for run()) into the reference's array formats.  dst holds n_trees * max_nodes * <row> elements; rows at or
   beyond a tree's size are filled with 0 (-1 for "trees").  */
#define MCTSNC_F_TREES 0            /* int32[T][max_nodes][1+A]: parent, children */
#define MCTSNC_F_SIZES 1            /* int32[T] */
#define MCTSNC_F_DEPTHS 2           /* int16[T][max_nodes] */
#define MCTSNC_F_TURNS 3            /* int8 [T][max_nodes] */
#define MCTSNC_F_LEAVES 4           /* uint8[T][max_nodes] */
#define MCTSNC_F_TERMINALS 5        /* uint8[T][max_nodes] */
#define MCTSNC_F_OUTCOMES 6         /* int8 [T][max_nodes] (2 = ongoing) */
#define MCTSNC_F_NS 7               /* int32[T][max_nodes] */
#define MCTSNC_F_NS_WINS 8          /* int32[T][max_nodes] */
#define MCTSNC_F_BOARDS 9           /* int8 [T][max_nodes][rows*cols] */
#define MCTSNC_F_EXTRA_INFOS 10     /* int8 [T][max_nodes][extra_info_memory] */
#define MCTSNC_F_NODES_SELECTED 11  /* int32[T] (last step) */
#define MCTSNC_F_SELECTED_PATHS 12  /* int32[T][2048+2] (last step; length in the last column) */
#define MCTSNC_F_ACTIONS_EXPANDED 13 /* int16[T][A+2] (last step, in the layout of the handle's variant) */
#define MCTSNC_F_PLAYOUT_OUTCOMES 14 /* int32[T][2] (last step) */
#define MCTSNC_F_PLAYOUT_OUTCOMES_CHILDREN 15 /* int32[T][A][2] (last step, ACP) */
int mctsnc_export(mctsnc_handle *h, int32_t search, int32_t field, void *dst, int64_t max_nodes);

/* The random streams of search `search` as uint64[n][2] (s0, s1); which = 0: playout streams, 1: the OCP
   child-pick streams (one per tree).  For tests of the generator (numba create_xoroshiro128p_states). */
int mctsnc_export_rng(mctsnc_handle *h, int32_t search, int32_t which, uint64_t *dst, int64_t n);

/* Launch shape and memory the library chose (threads per tree -- all blocks of a tree's cluster together --, blocks
   resident per SM, bytes allocated). */
int mctsnc_query(mctsnc_handle *h, int32_t *threads_per_tree, int32_t *blocks_per_sm, int32_t *sm_count,
                 int64_t *bytes_allocated);

/* Diagnostic, no counterpart in the reference: record every slice of the following batched Connect-4 launches that run
   through the work queue (more trees than blocks fit on the device): 4 int64 per slice -- tree, start and end of the
   slice in nanoseconds of the device's global timer, (SM id << 32) | steps run.  max_records = 0 switches it off.
   mctsnc_read_slices copies the records of the last launch to the host (after the launch has been waited for). */
int mctsnc_trace_slices(mctsnc_handle *h, int32_t max_records);
int mctsnc_read_slices(mctsnc_handle *h, int64_t *dst, int32_t max_records, int32_t *n_records);

/* One Connect-4 search that allocates nothing (no counterpart in the reference, whose searcher always allocates its
   device arrays in init_device_side_arrays).  For callers that cannot allocate device memory themselves: code running
   while a framework's caching allocator owns the device, services that forbid allocation after start-up, plug-ins that
   are handed a stream and buffers only.  Tree pools, random streams and bookkeeping live in one fixed array inside the
   library image (about 0.75 MB on every device that loads the library), hence the limits below; beyond them the call
   returns MCTSNC_E_CAPACITY.
   board/extra_info/turn: host, as for mctsnc_run.  out_device: DEVICE buffer of 3*7+4 int64 supplied by the caller:
   root_ns[7], actions_ns[7], actions_ns_wins[7] (indexed by action), then best_action, best_win_flag, best_n, best_n_wins.
   The result equals mctsnc_run on a freshly created handle with the same arguments.  Work is queued on `stream` and
   not waited for, except that the first call on a device, and any call with a new (seed, n_trees, n_playouts, variant),
   looks up the array's device address, prepares the seeded streams and synchronises: such a call has to come before
   any stream capture (nothing is said here about capturing the later ones).  The root is passed to the device as
   kernel arguments; no host memory of the caller is read after the call returns.  All calls share the one array: it
   is re-initialised at the start of every call, and calls whose GPU work overlaps (other streams, other host threads)
   race on it.  The host-side set-up (address look-up, stream cache) is serialised by a mutex inside the library, so
   threads driving different devices may call concurrently; each device has its own copy of the array. */
#define MCTSNC_STATIC_MAX_TREES 4
#define MCTSNC_STATIC_MAX_PLAYOUTS 256
#define MCTSNC_STATIC_MAX_STEPS 512
int mctsnc_search_c4_static(const int8_t *board, const int8_t *extra_info, int32_t turn, int32_t variant, int32_t n_trees,
                            int32_t n_playouts, int64_t steps, float ucb_c, uint64_t seed, int64_t *out_device, void *stream);

/* Exchange step of root-parallel search over the GPUs of one box without a collective library (no counterpart in the
   reference, which is single-GPU): in-place sum over `world` ranks of an int64 vector that lives on each rank's device --
   the partial sums of mctsnc_reduce_trees_device.  Every rank stores its vector into every peer's buffer (plain peer
   stores over NVLink), raises a flag there and adds up what arrived in its own buffer; remote memory is only written.
   One process per GPU: create() allocates the local buffer on `device` and returns its CUDA IPC handle
   (MCTSNC_EXCHANGE_HANDLE_BYTES bytes); the ranks exchange the handles by any means (the Python wrapper uses
   torch.distributed.all_gather_object) and pass all of them, in rank order, to connect().  connect(ex, NULL) maps every
   peer onto the local buffer (loop-back, for tests).  allreduce() queues two small kernels on `stream`; the wait for the
   peers' flags gives up after wait_limit polls of about a quarter of a microsecond each, sets MCTSNC_EXCHANGE_TIMEOUT in
   the status word (sticky; read with status(), which synchronises the stream) and leaves the values as they were.
   Every rank must make the same sequence of allreduce calls. */
#define MCTSNC_EXCHANGE_HANDLE_BYTES 64
#define MCTSNC_EXCHANGE_TIMEOUT 1
typedef struct mctsnc_exchange mctsnc_exchange;
int mctsnc_exchange_create(int32_t rank, int32_t world, int64_t n_values_max, int32_t device, mctsnc_exchange **out,
                           unsigned char *ipc_handle_out);
int mctsnc_exchange_connect(mctsnc_exchange *ex, const unsigned char *all_handles);
int mctsnc_exchange_allreduce(mctsnc_exchange *ex, int64_t *values_device, int64_t n, int32_t wait_limit, void *stream);
int mctsnc_exchange_status(mctsnc_exchange *ex, int32_t *status_out, void *stream);
int mctsnc_exchange_destroy(mctsnc_exchange *ex);

/* Text for a return code of any function above (cf. puct_cpp_cuda_error_string, src/puct/puct_gpu_v3_cpp.cu:483-485). */
const char *mctsnc_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif /* MCTSNC_B200_H */
