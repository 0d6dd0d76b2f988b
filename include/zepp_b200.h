/* C ABI of libzepp_b200.so: the B200-native expert-parallel MoE layer behind Zepp's API.
 *
 * Conventions: every entry point returns 0 on success and a non-zero code on failure
 * (zepp_last_error() gives the message of the calling thread's last failure); nothing throws or
 * aborts.  Pointers named *_dev are CUDA device pointers, `stream` is a cudaStream_t passed as
 * void*.  All work is enqueued on `stream`; no entry point synchronises the device unless it says
 * so.  One host thread per rank, one process per GPU (or several ranks of one process on one
 * GPU through zepp_rt_link_local, which is how single-GPU tests play every rank).
 *
 * Each declaration cites the reference interface it replaces (paths inside andronius-yang/zepp).
 */
#ifndef ZEPP_B200_H
#define ZEPP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct zepp_rt zepp_rt;
typedef struct zepp_layer zepp_layer;

const char* zepp_last_error(void);
int zepp_abi_version(void);

/* ---- runtime: symmetric arena + peer mapping -------------------------------------------------
 * Replaces init_shm / create_symmetric_tensor (src/pybind/module.cc:41-184, src/core/flux_shm.cc:61-150,
 * 397-403): one device arena per rank, exported as a CUDA IPC handle and mapped by every peer. */
int zepp_rt_create(int rank, int world, int device, size_t arena_bytes, zepp_rt** out);
int zepp_rt_destroy(zepp_rt* rt);
int zepp_rt_ipc_handle(zepp_rt* rt, void* blob64);                 /* 64-byte handle of this rank's arena */
int zepp_rt_open_peers(zepp_rt* rt, const void* blobs, int world); /* [world][64] handles, rank order */
int zepp_rt_link_local(zepp_rt** rts, int world);                  /* ranks of one process on one device */
int zepp_rt_set_wait_limit_ms(zepp_rt* rt, int ms);                /* bound of every device-side wait */
int zepp_rt_sm_count(zepp_rt* rt);

/* ---- layer ------------------------------------------------------------------------------------
 * zepp_layer_cfg mirrors EPMoEConfig + ModelShape (python/zepp/config.py:5-79) and Capacities
 * (python/zepp/routing.py:388-397). */
typedef struct {
  int32_t num_experts, topk, hidden, ffn_hidden;
  int32_t act;                 /* 0 gelu, 1 swiglu */
  int32_t ranks, ranks_per_node, max_tokens_per_rank;
  int32_t strategy;            /* 0 overlap (fused), 1 direct (unfused) */
  int32_t swap, redundant_slots_per_rank, sm_margin, gpu_plan;
  int64_t c_num, c_den;        /* router_c as an exact rational */
  int64_t caps[8];             /* recv_cap, dispatch_recv, dispatch_stage, dispatch_relay, combine_send,
                                  combine_conv, combine_wire, pair_cap */
} zepp_layer_cfg;

size_t zepp_layer_arena_bytes(const zepp_layer_cfg* cfg);
/* DispatchGemmOp + GemmCombineOp constructors (src/pybind/dispatch.cc:115-193, combine.cc:121-220) */
int zepp_layer_create(zepp_rt* rt, const zepp_layer_cfg* cfg, zepp_layer** out);
int zepp_layer_destroy(zepp_layer* layer);
/* Planner.apply_placement (python/zepp/planner.py:78-88): host tables p2l [R*nlp], l2p [G,R], lcnts [G] */
int zepp_layer_set_placement(zepp_layer* layer, const int32_t* p2l, const int32_t* l2p, const int32_t* lcnts,
                             void* stream);
/* OverlapComm.set_weights (python/zepp/comm/overlap.py:95-100): w1 [gpe, ffn1, H], w2 [gpe, H, ffn] bf16 */
int zepp_layer_set_weights(zepp_layer* layer, const void* w1_dev, const void* w2_dev);

/* Token buckets of the serving path (python/zepp/serving.py:42-50, 687-734: every rank pads its step to a common
 * bucket S_b <= max_tokens_per_rank): the following steps run at `tokens` rows per rank.  Every rank must choose
 * the same value.  Buffers keep their size; zepp_layer_step keeps one captured graph per (bucket, pointers).
 * Pad rows carry expert id -1 in topk_ids: such a copy has no owner, is counted in no load or split, moves no
 * row and is not computed (the reference routes pad rows to local experts and subtracts them from the loads
 * again, serving.py:147-160). */
int zepp_layer_set_tokens(zepp_layer* layer, int tokens);

/* WeightSlots (python/zepp/swap.py:236-300): with swap on, the layer owns the peer-visible weight slots
 * w1 [gpe, ffn1, H], w2 [gpe, H, ffn] that swapped experts travel between; callers fill them in place (or
 * pass their own tensors to zepp_layer_set_weights, which copies them in). */
int zepp_layer_weight_slots(zepp_layer* layer, void** w1_dev, void** w2_dev);

/* EPMoE.prepare (python/zepp/layer.py:145-171): loads exchange -> (swap decision + weight movement) ->
 * route -> routing exchange -> routed metadata, all on the device.  Phases: 0 loads, 1 swap decision and
 * pull of incoming experts (no-op with swap off), 2 commit of the pulled experts + route, 3 metadata;
 * zepp_layer_prepare runs all four (ranks in separate processes); linked single-process ranks call one
 * phase for every rank before the next phase. */
int zepp_layer_prepare(zepp_layer* layer, const int32_t* topk_ids_dev, const float* topk_weights_dev, void* stream);
int zepp_layer_prepare_phase(zepp_layer* layer, int phase, const int32_t* topk_ids_dev,
                             const float* topk_weights_dev, void* stream);
/* EPMoE.forward (python/zepp/layer.py:173-195): dispatch_gemm -> activation -> gemm_combine.
 * Phases: 0 publish x, 1 dispatch GEMM (+pull), 2 combine GEMM (+push), 3 top-k reduce into y. */
int zepp_layer_forward(zepp_layer* layer, const void* x_dev, void* y_dev, void* stream);
int zepp_layer_forward_phase(zepp_layer* layer, int phase, const void* x_dev, void* y_dev, void* stream);
/* prepare + forward in one call (what bench/replay.py:147-149 does per iteration).  topk_ids_dev and
 * topk_weights_dev are read in place by the step's kernels: keep them unchanged until the step ran. */
int zepp_layer_step(zepp_layer* layer, const int32_t* topk_ids_dev, const float* topk_weights_dev, const void* x_dev,
                    void* y_dev, void* stream);

/* Deferred verdict (src/core/verdict.h): synchronises `stream`, copies the 8 status words
 * (error bits, what/peer/epoch of a wait that gave up, violation mask) and clears the error bits. */
int zepp_layer_status(zepp_layer* layer, void* stream, uint64_t out[8]);
/* Device pointers of the planner products of the last prepare, for parity tests and host-planned
 * callers (what derive_routed_meta returns, src/pybind/dispatch.cc:159-167).  `which`: see ZEPP_T_*. */
int zepp_layer_table(zepp_layer* layer, int which, void** dev_ptr, size_t* bytes);
enum {
  ZEPP_T_LOADS = 0, ZEPP_T_PHYS_OWN = 1, ZEPP_T_VCE = 2, ZEPP_T_PROBS_ALL = 3, ZEPP_T_SPLITS = 4,
  ZEPP_T_SCATTER_INDEX = 5, ZEPP_T_SPS = 6, ZEPP_T_UC = 7, ZEPP_T_DEMANDS = 8, ZEPP_T_DPLAN = 9,
  ZEPP_T_CPLAN = 10, ZEPP_T_ROUTE_WS = 11, ZEPP_T_SWAP_BLOCK = 12, ZEPP_T_M_THIS = 13, ZEPP_T_ROW_TOK = 14,
  ZEPP_T_ACT = 15, ZEPP_T_RECV = 16, ZEPP_T_P2L = 17, ZEPP_T_L2P = 18, ZEPP_T_N_TILES = 19, ZEPP_T_PANEL = 20,
  ZEPP_T_GATE = 21, ZEPP_T_SCHED = 22
};
/* Device timeline of the last step (no counterpart in the reference, whose brackets are host-recorded events,
 * bench/replay.py:134-167): synchronises `stream` and copies 64 words (32..47 / 48..63: start / end stamps of the last 16 steps); words 8..19 are globaltimer ns stamps:
 * route, pass1, pass1 after its wait, pass2, dispatch GEMM start / x ready / end, combine GEMM start / end,
 * reduce start / after its wait / end. */
int zepp_layer_trace(zepp_layer* layer, void* stream, uint64_t out[64]);
int zepp_layer_gpu_launches(zepp_layer* layer, int64_t* out);  /* kernels launched so far by this layer */

/* ---- stand-alone planner entry points (one GPU plays every rank: they take R, L, my_rank) ------ */
/* route_workspace_ints (src/planner/routing.cu:572-575) and the word offsets inside it:
 * offs[10] = rep, rphys, c, D, U, Lb, fill, M, release, extra; stride of a replica table = min(R, 32) */
int zepp_route_workspace_ints(int G, int R);
int zepp_route_ws_offsets(int G, int R, int64_t offs[10]);
/* route / route_fused (src/pybind/routing.cc:9-78; src/planner/routing.cu:686-705): tables, budgets,
 * deterministic assignment, vacate, send row [phys | weight bits].  stats_dev int64[4]. */
int zepp_route(const int32_t* topk_own_dev, int S, int K, const int32_t* loads_dev, const int32_t* l2p_dev,
               const int32_t* lcnts_dev, int G, int R, int my_rank, int nlp, int L, int64_t c_num, int64_t c_den,
               int32_t* ws_dev, const float* probs_own_dev, int32_t* send_row_dev, int32_t* phys_own_dev,
               int64_t* stats_dev, void* stream);
/* planner_tail (src/planner/lane_device.cu:526-540) + routed_meta (src/pybind/dispatch.cc; kernels
 * src/dispatch/sort_util.cu:354-541): gathered [R, 2*S*K] or vce [R*S, K] -> splits, scatter_index, sps, uc,
 * demands[8] (a2av_demands, sort_util.cu:957-1122), dispatch plan head (a2av_dispatch_plan, :1153-1500),
 * combine tables (a2av_combine_tables, src/combine/combine_kernels.cu:1308).  Null outputs are skipped
 * except vce/splits/scatter_index/sps/uc/demands.  ws_dev: zepp_meta_workspace_bytes(). */
size_t zepp_meta_workspace_bytes(int R, int S, int K, int gpe);
int zepp_routed_meta(const int32_t* gathered_dev, const int32_t* vce_in_dev, int R, int L, int S, int K, int nlp,
                     int gpe, int my_rank, int direct, int relay_slots, const int64_t caps[8], int copies_per_rank,
                     int32_t* vce_dev, float* probs_all_dev, int32_t* splits_dev, int32_t* scatter_index_dev,
                     int32_t* sps_dev, int32_t* uc_dev, int64_t* demands_dev, int64_t* dplan_dev, int64_t* cplan_dev,
                     void* ws_dev, void* stream);
/* No counterpart in the reference.  zepp_routed_meta for callers that cannot allocate device memory where they
 * plan (a server whose own pool holds the whole GPU, a thread that must not block in the allocator): same
 * arguments minus the workspace; the scratch is a 1 MiB array inside the library image on every GPU that loads
 * it.  Routings whose scratch need (zepp_meta_workspace_bytes) exceeds 1 MiB are refused with an error.  Calls no
 * cudaMalloc / cudaFree.  The first call on a device looks up the array's address (make that call before any
 * stream capture, with the device current).  All calls on a device share the one array: two calls whose
 * kernels may overlap on the GPU (different streams) race; calls on one stream are safe. */
int zepp_routed_meta_noalloc(const int32_t* gathered_dev, const int32_t* vce_in_dev, int R, int L, int S, int K,
                             int nlp, int gpe, int my_rank, int direct, int relay_slots, const int64_t caps[8],
                             int copies_per_rank, int32_t* vce_dev, float* probs_all_dev, int32_t* splits_dev,
                             int32_t* scatter_index_dev, int32_t* sps_dev, int32_t* uc_dev, int64_t* demands_dev,
                             int64_t* dplan_dev, int64_t* cplan_dev, void* stream);
int zepp_dispatch_plan_words(int L, int NN);
/* swap_decide (src/planner/swap_decide.cu:81-346): rewrites p2l / l2p in place, fills the result block
 * int64[zepp_swap_decide_out_ints]. */
int zepp_swap_decide_out_ints(int R, int G, int nlp, int cap);
int zepp_swap_decide(const int32_t* loads_dev, int32_t* p2l_dev, int32_t* l2p_dev, const int32_t* lcnts_dev, int R,
                     int G, int L, int nlp, double C, int cap, int max_rounds, int64_t* out_dev, void* stream);
/* lane_arm (src/planner/lane_device.cu:49-80) */
int zepp_lane_arm(const int64_t* swap_out_dev, int R, int rank, int nlp, int cap, int64_t* gate_dev,
                  int32_t* sched_dev, int64_t* ovr0_dev, int64_t* ovr1_dev, const int64_t* stag_dev, int64_t epoch,
                  void* stream);
/* bounded 1-warp wait (src/core/cuda_common.cu:91-108 wait_geq_kernel): waits until *flag >= value or
 * limit_ms passed; result_dev[0] = 1 reached, 0 gave up.  Used to test the timeout path without a hang. */
int zepp_wait_geq(const uint64_t* flag_dev, uint64_t value, int limit_ms, int32_t* result_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif
