/*
 * coral_b200 -- C ABI of the B200 (sm_100a) batched graph beam search.
 *
 * Drop-in boundary for ONE path of the CORAL index: the batched "full expansion"
 * beam search behind IndexGPU::Search.  Plain pointers and sizes only; every
 * function returns a status code (0 = CORAL_OK), never exits the process and
 * never traps the device.  Each declaration cites the reference interface it
 * replaces (paths are relative to the reference project).
 *
 * Layout in device memory (owned by the handle unless attached):
 *   vectors    float  [n][dim]       row-major, rows are dim*4 bytes, dim % 4 == 0
 *   adjacency  int32  [n][deg_pad]   deg_pad = max_degree rounded up to 32/64/128,
 *                                    valid neighbour ids first, -1 padding
 *   start ids  int32  [M]
 * Distances follow the reference: L2 is the squared distance (no sqrt), IP is
 * the raw dot product and LARGER means closer (include/utils.cuh:254-323,380-382).
 */
#ifndef CORAL_B200_H
#define CORAL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* DIST_METRIC (include/uni.h) */
#define CORAL_L2 0
#define CORAL_IP 1

/* status codes */
#define CORAL_OK 0
#define CORAL_ERR_ARG 1      /* bad argument (null pointer, size out of range, dim % 4 != 0 ...) */
#define CORAL_ERR_STATE 2    /* call order: vectors/adjacency/start ids/prepare missing */
#define CORAL_ERR_CUDA 3     /* a CUDA runtime call failed; see coral_last_error */
#define CORAL_ERR_NOGPU 4    /* no usable CUDA device: there is no CPU fallback */
#define CORAL_ERR_KERNEL 5   /* the kernel gave up on a bounded wait; results are invalid */
#define CORAL_ERR_LIMIT 6    /* request exceeds what coral_search_prepare sized */
#define CORAL_ERR_QUERY 7    /* results are in place, but some query ended with a per-query status >= 2 */

/* per-query status written to stats[q][0] */
#define CORAL_Q_OK 0
#define CORAL_Q_BEAM_UNDERFULL 1  /* fewer than L nodes reachable (reference asserts, src/search_gpu.cu:444) */
#define CORAL_Q_HASH_OVERFLOW 2   /* visited set outgrew its tables: result approximate */
#define CORAL_Q_ROUND_LIMIT 3     /* stopped by the round bound */
#define CORAL_Q_BAD_START 4       /* a start id outside [0, n) was skipped (never dereferenced) */

/* stats row per query: status, n_dist, n_exp, rounds, hops, n_scan, max_cand, n_spill */
#define CORAL_STATS_W 8

typedef struct coral_index coral_index_t;

/* Library version and the SM architecture the kernels were compiled for (100). */
int coral_version(void);
int coral_compiled_sm(void);

/* The kernel's automatic shared-memory plan for vectors of `dim` floats and beam
 * capacity L on a device with `smem_optin_bytes` of opt-in shared memory per CTA
 * (232448 on B200): out8 = warps per CTA, CTAs per SM, bytes per row chunk, chunks
 * per row, stage buffers per warp, dynamic shared memory per CTA, candidate sort
 * tile, beam array length.  Pure host arithmetic (no device needed).  Replaces the
 * launch-shape arithmetic at src/search_gpu.cu:859-860. */
int coral_plan(int dim, int L, int smem_optin_bytes, int* out8);

/* Replaces the GPU branch of Graph::Graph (include/graph.cuh:222-266) and
 * GPUFuncs::GPUFuncs (src/gpufuncs.cu:70-118): binds a handle to `device`
 * and records the index geometry.  metric: CORAL_L2 | CORAL_IP. */
int coral_index_create(coral_index_t** out, int device, int64_t n, int dim, int max_degree, int metric);

/* Replaces RunFree / ~Graph: releases every device allocation of the handle. */
int coral_index_destroy(coral_index_t* h);

/* Replaces the base-vector cudaMemcpy at include/graph.cuh:260-261.  `vecs`
 * may be a host or a device pointer to n*dim floats; the data is copied. */
int coral_index_set_vectors(coral_index_t* h, const float* vecs);

/* Writes rows [first_row, first_row + count) of the handle's own vector array (allocating it for n
 * rows on first use): how vectors to be inserted later reach the device.  Replaces the copy in
 * Graph::insert_nodes (src/graph.cpp:277-279).  Host or device pointer. */
int coral_index_write_vectors(coral_index_t* h, int64_t first_row, int64_t count, const float* vecs);

/* Same, without the copy: `dev_vecs` must stay valid (and 16-byte aligned)
 * for the life of the handle.  No counterpart in the reference. */
int coral_index_attach_vectors(coral_index_t* h, const float* dev_vecs);

/* Replaces the Slot upload at include/graph.cuh:258-259.  Takes the graph as
 * the reference's Slot array presents it (include/disk_graph.h:30-35): for node
 * i, degs[i*deg_stride] neighbours at nbrs[i*nbr_stride + 0..deg).  Strides are
 * in int32 units (a Slot array is deg_stride = nbr_stride = 100).  Host
 * pointers.  Degrees above max_degree are cut (src/graph.cu:723-727). */
int coral_index_set_slots(coral_index_t* h, const int32_t* degs, size_t deg_stride,
                          const int32_t* nbrs, size_t nbr_stride);

/* The same graph already in the padded device layout: int32 [n][deg_pad], -1
 * padding.  Host or device pointer; copied. */
int coral_index_set_adjacency(coral_index_t* h, const int32_t* adj, int deg_pad);

/* Replaces Graph::load_search_start_nodes / get_start_ids
 * (src/graph.cpp:329-351): all M ids are used as entry points, duplicates kept
 * (src/search_gpu.cu:392-407). */
int coral_index_set_start_ids(coral_index_t* h, const int32_t* ids, int M);

/* Replaces Graph::FPS (src/start.cu:72-145): picks M entry points by
 * farthest-point sampling over BFS hop counts on the installed adjacency and
 * installs them as with coral_index_set_start_ids.  ids[0] = first_id; each
 * further id is the lowest-numbered node whose smallest hop count from the
 * ids chosen so far is largest (a node no chosen id reaches counts as -1).
 * The reference draws the first node at random until it has an out-edge
 * (src/start.cu:77-86); here the caller names it, so the same graph gives the
 * same ids, and a first_id without out-edges is CORAL_ERR_ARG.  ids_out
 * (host, M ints) may be NULL.  Needs 16 bytes of device scratch per node,
 * freed before returning. */
int coral_index_select_start_ids(coral_index_t* h, int first_id, int M, int32_t* ids_out);

/* The handle's own stream (a cudaStream_t, created non-blocking): what NULL stream arguments of
 * this library mean.  Replaces GPUFuncs::get_stream (include/gpufuncs.cuh:607). */
void* coral_index_stream(coral_index_t* h);

/* Reads the installed graph back: adjacency [n][deg_pad] to a host or device buffer (replaces the
 * device-to-host copy of Graph::write_back_all_gpu_slots behind save_build, include/graph.cuh:481),
 * and the entry points (returns how many are installed; copies at most `capacity` to ids_out, which
 * may be NULL) as Graph::get_start_ids does (include/graph.cuh:494). */
int coral_index_get_adjacency(coral_index_t* h, int32_t* adj_out);
int coral_index_get_start_ids(coral_index_t* h, int32_t* ids_out, int capacity);

/* Replaces d_deleted (src/search_gpu.cu:582-833, :716): bit i set = node i is
 * skipped when the final top-k is written.  Host pointer to (n+31)/32 words, or
 * NULL to clear. */
int coral_index_set_deleted(coral_index_t* h, const uint32_t* bits);

/* Replaces GPUFuncs::search_prepare (src/search.cu:400-440): sizes every
 * scratch buffer once for up to max_queries per call, beam capacity <= max_L
 * and k <= max_k.  The reference reallocates on every Search. */
int coral_search_prepare(coral_index_t* h, int max_queries, int max_L, int max_k);

/* Replaces GPUFuncs::search_free (src/search.cu:442-456). */
int coral_search_free(coral_index_t* h);

/* Replaces IndexGPU::Search (src/index_gpu.cpp:117-136) + GPUFuncs::search_gpu
 * (src/search_gpu.cu:835-886).  queries: Q*dim floats, ids_out: Q*k int32,
 * dists_out (may be NULL): Q*k floats, stats_out (may be NULL): Q*CORAL_STATS_W
 * int32 -- each a HOST or a DEVICE pointer (detected).  L = beam capacity,
 * k <= L, M = number of start ids <= L.  Blocks until results are in place.
 * total_hops_out (may be NULL) receives the reference's Test_Result::hops. */
int coral_search(coral_index_t* h, const float* queries, int Q, int L, int k, int32_t* ids_out,
                 float* dists_out, int32_t* stats_out, int64_t* total_hops_out);

/* The kernel window alone: all pointers are device pointers, the launch is
 * enqueued on `stream` (a cudaStream_t, NULL = the handle's stream) and the
 * call returns without synchronising.  Check coral_search_check afterwards. */
int coral_search_async(coral_index_t* h, const float* d_queries, int Q, int L, int k,
                       int32_t* d_ids_out, float* d_dists_out, int32_t* d_stats_out, void* stream);

/* The order in which a large batch is run for locality: d_order_out[i] (device, Q ints) = the row of
 * the i-th query to run, the batch sorted by each query's closest neighbour of the entry points,
 * equal keys in row order (deterministic: every GPU that orders the same batch over the same
 * replicated index gets the same order, so rank r of a replicated multi-GPU search can take the
 * r-th contiguous range of the ORDERED batch and see 1/world of the graph at full multiplicity).
 * The query x frontier scores are the dense contraction of this path and run on the tensor cores
 * (replaces nothing in the reference, whose warp_calc_dist seeds one start node per warp,
 * src/search_gpu.cu:14-23).  Enqueued on `stream` (NULL = the handle's), no synchronisation. */
int coral_query_order(coral_index_t* h, const float* d_queries, int Q, int32_t* d_order_out, void* stream);

/* After the stream has been synchronised: CORAL_ERR_KERNEL if the last launch
 * reported a bounded wait that ran out, else CORAL_OK. */
int coral_search_check(coral_index_t* h);

/* Device time in milliseconds of the last coral_search's kernel window (the
 * reference's timed window, src/search_gpu.cu:861-877) and of the whole call. */
float coral_last_kernel_ms(coral_index_t* h);
float coral_last_total_ms(coral_index_t* h);

/* Number of kernels this library launched on behalf of the handle so far. */
int64_t coral_launch_count(coral_index_t* h);

/* Tuning knobs (set before coral_search_prepare; none of them changes a result):
 *   "ctas_per_sm", "warps"   resident CTAs per SM and warps per CTA; 0 = automatic (the warps in
 *                            3..6 that keep most warps resident; 8 warps for batches <= 4 x SMs)
 *   "chunk_bytes"            bytes of a row moved by one bulk copy; 0 = automatic (256, or up to
 *                            512 when the row does not split into 256-byte chunks and five CTAs
 *                            still fit an SM)
 *   "stages"                 stage buffers per warp; 0 = automatic (1)
 *   "gather"                 how row chunks reach shared memory: 0 = one bulk copy per row chunk,
 *                            1 = 16-byte cp.async units, 2 = one tensor copy per four rows (a tensor map
 *                            of the row array, chunk width an odd number of 16-byte units, 272 bytes
 *                            unless "chunk_bytes" says otherwise); -1 = automatic (default): 2 when the
 *                            driver's tensor-map encoder is available, else 0
 *   "smem_hash_bits"         log2 entries of a shared-memory visited table in front of the global
 *                            one; 0 = none (default)
 *   "visit_cache_bits"       log2 entries of a shared-memory cache of recently seen ids; 0 = none
 *   "ghash_factor", "ghash_entries"   global visited table per CTA: >= factor x L x deg_pad
 *                            entries (default 8), or an explicit power of two >= 64
 *   "sort_tile"              candidate keys sorted at once at the end of a round; 0 = automatic
 *                            (about twice the beam capacity)
 *   "scout_ids"              neighbour ids a lane examines per scout step, 1..4; 0 = automatic
 *   "max_rounds"             per-query round limit (status 3 when reached)
 *   "cluster_size"           CTAs that share one query when the batch is far smaller than the GPU:
 *                            0 = automatic, 1 = never, 2/4/8/16 = forced
 *   "schedule_tc"            scheduling keys on the tensor cores (1, default) or by fp32 SIMT tiles (0)
 *   "dense_passes"           tf32 passes of coral_exact_knn's selection scans: 3 (default) or 1
 *   "schedule"               run large batches grouped by the entry points' neighbour each query is
 *                            closest to, for L2 locality: 0 = automatic for batches >= 8192,
 *                            1 = always, -1 = never
 * coral_get_option also answers "plan_stages", "plan_warps", "plan_chunk_bytes",
 * "plan_smem_bytes", "plan_hash_bits", "plan_ctas_per_sm" (the plan of the most recent search or
 * prepare), "last_cluster_size", "last_scheduled", "frontier_size", "grid_cap", "deg_pad", "dim".
 * Returns CORAL_ERR_ARG for unknown names. */
int coral_set_option(coral_index_t* h, const char* name, int value);
int coral_get_option(coral_index_t* h, const char* name, int* value);

/* Replaces ids_verify_kernel / GPUFuncs::search_verify
 * (src/search_gpu.cu:888-922): hits = sum_q |res[q][0..k) ∩ gt[q][0..k)|, gt rows
 * are gt_dim wide (tests/test_search_pipeline.cpp:25-39).  Host or device
 * pointers. */
int coral_count_hits(coral_index_t* h, const int32_t* res, const int32_t* gt, int Q, int k,
                     int gt_dim, int64_t* hits_out);

/* Replaces the exhaustive Faiss flat search the reference calls for the k_b nearest
 * base points of its training queries (src/knn.cu:174-193, include/myfaiss.h:17-29)
 * and for ground truth (tests/comp_gt.cpp:121-155): the k closest of the handle's
 * vectors for each of Q queries, closest first, ties by the smaller id.  The scores
 * are formed on the tensor cores (tcgen05, tf32 operands split into high and low
 * parts, three passes: fp32-grade) and only SELECT the k + 28 best per query; those
 * are re-ranked with the exact fp32 distance in the order of the reference's device
 * functions (include/utils.cuh:254-275, :307-323), which is also what dists_out
 * (nullable) receives.  A query is certified when its exact k-th distance beats the
 * best score an unselected row could have; *uncertified_out (nullable) counts the
 * others (their answer is almost surely right, but not proven).  k <= 228.  Host or
 * device pointers.  Option "dense_passes" = 1 selects with one plain tf32 pass. */
int coral_exact_knn(coral_index_t* h, const float* queries, int Q, int k, int32_t* ids_out,
                    float* dists_out, int64_t* uncertified_out);

/* Device time (ms) and tensor-core floating-point operations (2 x passes x Q x n x dim)
 * of the last coral_exact_knn call: selection scans and re-rank. */
float coral_last_dense_ms(coral_index_t* h);
double coral_last_dense_flops(coral_index_t* h);

/* ---- graph build (the callers of the search path on the build side) ----
 *
 * Replaces the HBM-tier build of IndexGPU::BuildGPU (src/index_gpu.cpp:308-383): the exact
 * nearest-neighbour lists of the training queries (coral_exact_knn) are projected onto the base
 * set batch by batch (coral_build_nap), then nodes no list reached are connected by searching
 * the partial graph with their own vector (coral_build_connect_enhance).  The graph lives in
 * the handle's adjacency, so it can be searched at any point; rows are kept closest-first with
 * the distance of every edge, like the reference's Slot (include/disk_graph.h:30-35).  Where
 * the reference lets thread arrival order decide (src/upd_gpu.cu:102, src/enhance.cu:166) the
 * lowest index wins, so a build is reproducible. */

/* Replaces Graph::Graph in Mode::CONS (include/graph.cuh:222-266): an empty graph over the
 * handle's vectors (every degree 0); allocates the edge distances and build scratch. */
int coral_build_begin(coral_index_t* h);

/* Replaces GPUFuncs::graph_update / gpu_neibor_aware (src/upd_disk.cu:218, src/upd_gpu.cu:260-303)
 * for T lists of kb base ids (host or device, row-major), `batch` lists at a time (0 = 1024,
 * config.json:5): per list member, candidates = the other members (skipping pairs of already
 * connected nodes) + its current neighbours, sorted by distance, occlusion-pruned, kept ones
 * first then pruned ones up to max_degree.  2 <= kb <= 128, kb + max_degree <= 256. */
int coral_build_nap(coral_index_t* h, const int32_t* lists, int T, int kb, int batch);

/* Replaces GPUFuncs::gpu_connect_enhance, enhance_mode 0 (src/enhance.cu:728-812): every node
 * of degree 0, in batches of `search_batch` (0 = 524288), is searched with its own vector
 * (beam capacity L, 0 = 256; kb results) from M (0 = 16) entry points chosen per batch by
 * coral_index_select_start_ids from the lowest-numbered connected node; then, `nap_batch`
 * (0 = 4096) nodes at a time, the found nodes receive a reverse edge (src/enhance.cu:136-212)
 * and the node gets its own pruned row.  Calls coral_search_prepare (sizes: search_batch, L,
 * kb) and leaves the last batch's entry points installed, as the reference's save_build does.
 * The reference's second phase ("top hit" nodes, src/enhance.cu:814-856) is not built. */
int coral_build_connect_enhance(coral_index_t* h, int kb, int L, int search_batch, int nap_batch, int M,
                                int64_t* n_isolated_out);

/* Reads / replaces the graph under construction: adjacency [n][deg_pad] (-1 padding), edge
 * distances [n][deg_pad], degrees [n]; host or device pointers, NULL = skip (get only).
 * Replaces Graph::save_build / load (include/graph.cuh:481-484) at the C boundary. */
int coral_build_get_graph(coral_index_t* h, int32_t* adj_out, float* dists_out, int32_t* degs_out);
int coral_build_set_graph(coral_index_t* h, const int32_t* adj, const float* dists, const int32_t* degs);

/* ---- update: delete with topology repair, insert (src/index_gpu.cpp:138-224) ----
 * Rows [0, live) of the vector array are the index; rows [live, n) hold vectors that are not
 * inserted yet (the reference keeps inserted vectors behind the base the same way,
 * src/graph.cpp:264-287).  coral_index_set_live declares `live` before a build over a prefix. */
int coral_index_set_live(coral_index_t* h, int64_t live);

/* Enters update mode on a searchable index: computes the distance of every stored edge and the
 * degrees (the reference keeps them in its Slot, include/disk_graph.h:34) unless a build is still
 * open.  Leave with coral_build_end. */
int coral_build_begin_from_graph(coral_index_t* h);

/* Replaces IndexGPU::Delete (src/index_gpu.cpp:138-206) + GPUFuncs::vector_delete
 * (src/update.cu:674-771): marks `count` ids (host) deleted -- the bitset of
 * coral_index_set_deleted -- finds their live in-neighbours on the GPU (the reference keeps host
 * hash sets, src/graph.cpp:139-195), and repairs every in-neighbour in batches of 131072: its
 * surviving neighbours plus the deleted node's surviving out-neighbours, sorted closest-first,
 * occlusion-pruned, kept ones first then pruned ones.  The first (deleted node, in-neighbour) pair
 * of a batch repairs an in-neighbour (reference: thread arrival); in-neighbours are taken in
 * ascending id order.  Then M entry points (0 = as many as installed) are chosen again
 * (coral_index_select_start_ids) from the lowest-numbered live, undeleted, connected node. */
int coral_delete(coral_index_t* h, const int32_t* ids, int count, int M);

/* Replaces IndexGPU::Insert (src/index_gpu.cpp:207-224) + GPUFuncs::vector_insert with neighbours
 * from the search (src/update.cu:880-959, upd_type 1): rows [first_id, first_id + count) --
 * first_id must be the current live count -- become nodes, `batch` (0 = 2048) at a time: entry
 * points re-chosen, each new vector searched with beam capacity L (0 = 512) for kb neighbours,
 * reverse edges into the found nodes (src/update.cu:143-191), the new node's own row from its
 * pruned candidates.  Calls coral_search_prepare (batch, L, kb). */
int coral_insert(coral_index_t* h, int64_t first_id, int count, int kb, int L, int batch, int M);

/* Replaces GPUFuncs::Build_Free: releases the edge distances and build scratch; the adjacency
 * (and the installed entry points) stay for searching. */
int coral_build_end(coral_index_t* h);

/* Shard merge (no counterpart in the reference, which is single-GPU): ids and
 * dists hold G per-shard results [G][Q][k] (global ids, -1 = padding); writes
 * the k closest per query by (distance, id).  Device pointers; enqueued on
 * `stream` without synchronising. */
int coral_merge_shards(coral_index_t* h, const int32_t* d_ids, const float* d_dists, int G, int Q,
                       int k, int32_t* d_ids_out, float* d_dists_out, void* stream);

/* The same with the G per-shard blocks `shard_stride` elements apart (>= Q*k): merges a
 * slice of a larger gathered buffer in place.  No counterpart in the reference. */
int coral_merge_shards_strided(coral_index_t* h, const int32_t* d_ids, const float* d_dists, int G,
                               int Q, int k, int64_t shard_stride, int32_t* d_ids_out,
                               float* d_dists_out, void* stream);

/* Maps shard-local result ids to global ids in place through id_map[n_local]
 * (device pointers; ids < 0 stay).  No counterpart in the reference. */
int coral_map_ids(coral_index_t* h, int32_t* d_ids, int64_t count, const int32_t* d_id_map, void* stream);

/* ---- multi-GPU (no counterpart in the reference, which drives one GPU: src/gpufuncs.cu:35,84;
 * its tiers for bases beyond one GPU are host memory and SSD, src/index_gpu.cpp:256-257) ----
 *
 * One handle per GPU.  An index that fits one GPU is replicated and the batch split: rank r of
 * `world` searches rows [lo, hi) of the batch (coral_query_slice) with plain coral_search -- no
 * collective.  An index that does not fit is sharded: every rank holds one shard (own graph,
 * own entry points, id_map[local] = global id), searches ALL queries, and coral_search_sharded
 * exchanges the per-shard top-k with ONE ncclAllGather and merges this rank's slice only.
 * NCCL is loaded with dlopen("libnccl.so.2") at the first coral_comm_* call. */
typedef struct coral_comm coral_comm_t;

/* 128-byte NCCL unique id for coral_comm_create (make it on one rank, hand it to the others). */
int coral_comm_unique_id(void* id128);
/* One communicator per process and GPU (collective: every rank must call it). */
int coral_comm_create(coral_comm_t** out, int device, int world, int rank, const void* id128);
/* n communicators for n GPUs driven by ONE process (out: n pointers); ranks = positions. */
int coral_comm_create_all(coral_comm_t** out, const int* devices, int n);
/* Installs this rank's local -> global id map (count ints, host or device; copied): used by
 * coral_search_sharded when its d_id_map argument is NULL. */
int coral_comm_set_id_map(coral_comm_t* c, const int32_t* ids, int64_t count);
int coral_comm_destroy(coral_comm_t* c);
int coral_comm_world(coral_comm_t* c);
int coral_comm_rank(coral_comm_t* c);
const char* coral_comm_last_error(coral_comm_t* c);

/* Rows [*lo, *hi) of a Q-query batch that `rank` of `world` owns (contiguous, balanced). */
void coral_query_slice(int Q, int world, int rank, int* lo, int* hi);

/* Sharded search, collective over the communicator: the same Q queries (host or device pointer) on
 * every rank.  Local search (as coral_search_async) -> global ids through d_id_map (device; NULL =
 * the map installed with coral_comm_set_id_map, or global ids already) -> one ncclAllGather of ids and distances in a single buffer
 * -> merge by (distance, id) of THIS rank's slice of the batch (coral_query_slice): ids_out /
 * dists_out (nullable) receive (hi - lo) * k entries, host or device pointers.  Everything is
 * enqueued on `stream` (NULL = the handle's stream); the call synchronises only when it has to
 * copy to host buffers.
 * Communication buffers are grown on demand and kept.  world * k <= 4096. */
int coral_search_sharded(coral_index_t* h, coral_comm_t* c, const int32_t* d_id_map, const float* d_queries,
                         int Q, int L, int k, int32_t* ids_out, float* dists_out, void* stream);

/* The beam search for callers that cannot allocate device memory at search time
 * (a server whose pool already owns the GPU, a plugin inside another framework's
 * callback, code under an allocation guard).  It has no counterpart in the
 * reference, whose Search allocates on every call (src/index_gpu.cpp:117-136).
 * Same kernel and same results as coral_search, but the kernel's scratch (visited
 * table, candidate buffers) lives in a 64 MiB array inside the library image, so
 * this function calls no cudaMalloc/cudaFree and builds no host containers.
 * Every pointer is a device pointer owned by the caller (a host pointer is
 * CORAL_ERR_ARG); adjacency is the padded layout [n][deg_pad].  Limits:
 * L * deg_pad <= 16384 (CORAL_ERR_LIMIT beyond), Q <= 2^24.  The first call on a
 * device resolves the array's address: make it before any stream capture.  All
 * calls share the array, which keeps the last call's contents (control words are
 * re-zeroed, table entries are epoch-tagged); calls that overlap on one GPU race.
 * Runs on `stream` and returns after synchronising it.
 * Differences from coral_search: there is no per-query stats array; instead the
 * worst per-query status of the call is kept (coral_search_static_status), and a
 * call in which some query ended with status >= CORAL_Q_HASH_OVERFLOW returns
 * CORAL_ERR_QUERY with the results in place.  A start id outside [0, n) is
 * skipped, never dereferenced (CORAL_Q_BAD_START).  The visited table per CTA has
 * 8 x L x deg_pad entries, as on the regular path, when a full grid fits the
 * array, else 4 x. */
int coral_search_static(int device, void* stream, const float* d_vecs, const int32_t* d_adj, int64_t n,
                        int dim, int deg_pad, int metric, const int32_t* d_start_ids, int M,
                        const float* d_queries, int Q, int L, int k, int32_t* d_ids_out, float* d_dists_out);

/* Worst per-query status (CORAL_Q_*) of the last coral_search_static call on
 * `device`; -1 for a device index out of range.  No counterpart in the reference. */
int coral_search_static_status(int device);

/* Last error text of the handle (or of handle creation when h is NULL). */
const char* coral_last_error(coral_index_t* h);

#ifdef __cplusplus
}
#endif
#endif /* CORAL_B200_H */
