// Host side of libzepp_b200.so: symmetric arena + peer mapping, the layer object, kernel launches
// and the extern "C" entry points declared in include/zepp_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/zepp_b200.h"
#include "common.cuh"
#include "front.cuh"
#include "gemm.cuh"
#include "gemm_pair.cuh"
#include "layer_kernels.cuh"
#include "meta.cuh"
#include "planner.cuh"
#include "swap.cuh"

using namespace zepp;

constexpr int kSwapCap = 8;        // expert moves per rank and step (the reference's SWAP_MAX_MOVES)

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
static thread_local std::string g_err;

static int fail(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return 1;
}

#define CU_OK(expr)                                                                         \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) return fail("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

static int swap_decide_prepare();
static SwapArgs swap_args(const int* loads, int* p2l, int* l2p, const int* lcnts, int R, int G, int L, int nlp, double C,
                          int cap, int max_rounds, long long* out);
static size_t swap_smem(int R, int G, int L, int nlp);
static size_t meta_smem(int R, int NN, int E_virt);
static size_t pass2_smem(int tokens_per_tile, int K, int E_virt);
static int pass2_prepare(size_t bytes);
static int meta_fused_prepare(zepp_layer* l);
static int front_push_blocks(const zepp_layer* l, int n_route);
static int pair_kernels_prepare(zepp_layer* l);
static void choose_gemm_kind(zepp_layer* l);

extern "C" const char* zepp_last_error(void) { return g_err.c_str(); }
extern "C" int zepp_abi_version(void) { return 1; }

// ---------------------------------------------------------------------------------------------
// runtime
// ---------------------------------------------------------------------------------------------
struct zepp_rt {
  int rank = 0, world = 1, device = 0, sm_count = 0;
  uint8_t* arena = nullptr;
  size_t arena_bytes = 0, bump = 0;
  uint8_t* peer_base[kMaxRanks] = {};
  bool opened[kMaxRanks] = {};
  bool peers_ready = false;
  unsigned long long wait_ns = 4000000000ull;
};

static void* rt_alloc(zepp_rt* rt, size_t bytes, size_t align = 1024) {
  size_t off = (rt->bump + align - 1) / align * align;
  if (off + bytes > rt->arena_bytes) return nullptr;
  rt->bump = off + bytes;
  return rt->arena + off;
}
template <typename T>
static T* peer_ptr(zepp_rt* rt, int p, T* local) {
  return reinterpret_cast<T*>(rt->peer_base[p] + (reinterpret_cast<uint8_t*>(local) - rt->arena));
}

extern "C" int zepp_rt_create(int rank, int world, int device, size_t arena_bytes, zepp_rt** out) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail("bad rank/world %d/%d", rank, world);
  CU_OK(cudaSetDevice(device));
  zepp_rt* rt = new (std::nothrow) zepp_rt();
  if (!rt) return fail("out of host memory");
  rt->rank = rank;
  rt->world = world;
  rt->device = device;
  cudaDeviceProp prop;
  CU_OK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    delete rt;
    return fail("libzepp_b200 needs an sm_100 device (found sm_%d%d)", prop.major, prop.minor);
  }
  rt->sm_count = prop.multiProcessorCount;
  rt->arena_bytes = (arena_bytes + 4095) / 4096 * 4096;
  cudaError_t e = cudaMalloc(&rt->arena, rt->arena_bytes);
  if (e != cudaSuccess) {
    delete rt;
    return fail("cudaMalloc of the %zu-byte arena failed: %s", arena_bytes, cudaGetErrorString(e));
  }
  CU_OK(cudaMemset(rt->arena, 0, rt->arena_bytes));
  rt->peer_base[rank] = rt->arena;
  rt->peers_ready = (world == 1);
  *out = rt;
  return 0;
}

extern "C" int zepp_rt_destroy(zepp_rt* rt) {
  if (!rt) return 0;
  cudaSetDevice(rt->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < rt->world; ++p)
    if (rt->opened[p]) cudaIpcCloseMemHandle(rt->peer_base[p]);
  if (rt->arena) cudaFree(rt->arena);
  delete rt;
  return 0;
}

extern "C" int zepp_rt_ipc_handle(zepp_rt* rt, void* blob64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  CU_OK(cudaSetDevice(rt->device));
  CU_OK(cudaIpcGetMemHandle(&h, rt->arena));
  memcpy(blob64, &h, 64);
  return 0;
}

extern "C" int zepp_rt_open_peers(zepp_rt* rt, const void* blobs, int world) {
  if (world != rt->world) return fail("open_peers: world %d != %d", world, rt->world);
  CU_OK(cudaSetDevice(rt->device));
  for (int p = 0; p < world; ++p) {
    if (p == rt->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, reinterpret_cast<const uint8_t*>(blobs) + 64 * p, 64);
    void* ptr = nullptr;
    CU_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    rt->peer_base[p] = reinterpret_cast<uint8_t*>(ptr);
    rt->opened[p] = true;
  }
  rt->peers_ready = true;
  return 0;
}

extern "C" int zepp_rt_link_local(zepp_rt** rts, int world) {
  for (int r = 0; r < world; ++r) {
    if (rts[r]->world != world || rts[r]->rank != r) return fail("link_local: runtime %d is rank %d of %d", r, rts[r]->rank, rts[r]->world);
    if (rts[r]->device != rts[0]->device) return fail("link_local: all ranks must be on one device");
    if (rts[r]->arena_bytes != rts[0]->arena_bytes) return fail("link_local: arena sizes differ");
  }
  for (int r = 0; r < world; ++r) {
    for (int p = 0; p < world; ++p) rts[r]->peer_base[p] = rts[p]->arena;
    rts[r]->peers_ready = true;
  }
  return 0;
}

extern "C" int zepp_rt_set_wait_limit_ms(zepp_rt* rt, int ms) {
  if (ms < 1) return fail("wait limit must be >= 1 ms");
  rt->wait_ns = (unsigned long long)ms * 1000000ull;
  return 0;
}
extern "C" int zepp_rt_sm_count(zepp_rt* rt) { return rt->sm_count; }

// ---------------------------------------------------------------------------------------------
// tensor maps
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// bf16 row-major [rows, cols]; box = 64 columns (128 bytes) x box_rows, 128-byte swizzle, zero fill
static int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (cols * 2) % 16 != 0) return fail("tensor map: unaligned base/stride");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu box %u)", (int)r,
                                     (unsigned long long)rows, (unsigned long long)cols, box_rows);
  return 0;
}

// ---------------------------------------------------------------------------------------------
// layer
// ---------------------------------------------------------------------------------------------
struct zepp_layer {
  zepp_rt* rt = nullptr;
  zepp_layer_cfg cfg{};
  int G, K, H, I, ffn1, W, L, NN, S, SK, nlp, gpe, E_virt, cap, max_tiles, tokens_per_tile, tiles_per_src;
  int S_max;                                  // tokens per rank the buffers were sized for (S: the current bucket)
  bool use_pairs = false;                     // the GEMMs run on CTA pairs (256-row token tiles)
  int pairs_mode = -1;                        // ZEPP_B200_PAIRS: 1 / 0 force the pair kernels on / off, -1 = by row count
  int pair_grid = 0;                          // CTAs of a pair-kernel launch (2 x resident clusters)
  bool meta_fused = false;                    // the metadata runs as one cooperative launch (grid fits the device)
  unsigned long long epoch = 0;
  int64_t launches = 0;
  bool have_weights = false, have_placement = false;
  // symmetric (peer-visible) buffers
  int* loads_all[2];                 // [R, G]
  int* xchg_all[2];                  // [R, 2*SK]
  unsigned long long *loads_flags, *routing_flags, *x_flags, *done_flags;   // [R] each
  __nv_bfloat16* xsym[2];            // [S, H]
  __nv_bfloat16* stage = nullptr;    // [W, S, H] staged dispatch rows, region s written by rank s
  unsigned long long* push_flags = nullptr;   // [R]
  __nv_bfloat16* panel;              // [S*K, H]
  // local buffers
  __nv_bfloat16 *recv, *act, *staging;
  int *slot_of, *topk_own, *phys_own, *send_row, *route_ws, *p2l, *l2p, *lcnts;
  float* probs_own;
  long long* route_stats;
  int *vce, *splits, *scatter_index, *sps, *uc, *tile_hist, *tile_uc, *expert_base;
  float* probs_all;
  long long *demands, *dplan, *cplan, *swap_block, *gate, *ovr0, *ovr1, *stag;
  int *sched, *redirect;
  int *n_tiles, *tile_group, *tile_row0, *tile_rows, *m_this, *row_tok;
  unsigned int *tile_ready, *counters;
  long long* row_dst;
  float* row_scale;
  unsigned long long* status;
  // device pointer tables
  const __nv_bfloat16** x_ptrs[2];
  // swap: weight slots owned by the layer (peer-visible) with the staging groups of incoming experts behind them
  __nv_bfloat16 *w1_slots = nullptr, *w2_slots = nullptr;     // [gpe + kSwapCap][...]
  const uint4 **w1_peers = nullptr, **w2_peers = nullptr;
  unsigned int* w_ready = nullptr;                            // [2 * kSwapCap] chunk counters of the staging entries
  const __nv_bfloat16** stage_ptrs = nullptr;   // [W] this rank's staging regions (one per source)
  PeerTable stage_dst, push_flag_dst;
  __nv_bfloat16** panels;
  unsigned long long** done_ptrs;
  // host peer tables for the publishing kernels
  PeerTable loads_dst[2], xchg_dst[2], loads_flag_dst, routing_flag_dst, x_flag_dst;
  // tensor maps
  CUtensorMap tm_w1, tm_w2, tm_recv[3], tm_act[3];
  const void* x_self = nullptr;
  const int* ids_in = nullptr;
  const float* wts_in = nullptr;
  unsigned long long* step_ctr = nullptr;     // device-resident step counter (epoch of the running step)
  int c_max = 1;                              // largest replica count of the resident placement
  bool use_graphs = true;
  bool combine_lines = false;                 // combine epilogue writes staged 128-byte lines
  const void* fuse_x = nullptr;       // x of a whole-step call, published by the routing kernel
  const void* x_fused = nullptr;
  cudaStream_t capture_stream = nullptr;
  // whole-step calls: roles the front kernel takes over from their stand-alone kernels (set per enqueue)
  bool front_route = false, front_push = false;
  int front_blocks_max = 0;                   // blocks of the front kernel the device keeps resident at once
  struct StepGraph {
    const void *ids, *wts, *x, *y;
    int tokens;                              // the bucket the launches were recorded for
    cudaGraphExec_t exec;
    int64_t kernels;
  };
  std::vector<StepGraph> graphs;
};

static size_t al(size_t v) { return (v + 1023) / 1024 * 1024; }

extern "C" size_t zepp_layer_arena_bytes(const zepp_layer_cfg* c) {
  const size_t R = c->ranks, G = c->num_experts, K = c->topk, H = c->hidden, I = c->ffn_hidden, S = c->max_tokens_per_rank;
  const size_t SK = S * K, nlp = G / R + c->redundant_slots_per_rank, gpe = nlp + 1, E = R * gpe, cap = c->caps[0];
  const size_t tiles = (SK + 1023) / 1024 + 1;
  size_t b = 0;
  b += 2 * al(R * G * 4) + 2 * al(R * 2 * SK * 4) + 6 * al(R * 8) + 2 * al(S * H * 2) + al(SK * H * 2);
  if (R > 1 && c->strategy == 0) b += al(R * S * H * 2);
  if (c->swap) b += (gpe + 8) * (al((c->act == 1 ? 2 : 1) * I * H * 2) + al(H * I * 2)) + (1 << 20);
  b += al(cap * H * 2) * 2 + al(cap * I * 2);
  b += 4 * al(SK * 4) + al(2 * SK * 4) + al((size_t)zepp_route_workspace_ints((int)G, (int)R) * 4);
  b += 3 * al(R * nlp * 4) + 2 * al(G * R * 4) + al(G * 4);
  b += 3 * al(R * SK * 4) + al(E * 4) + al(R * E * 4) + al(R * (2 * R) * 4);
  b += al(R * tiles * E * 4) + al(R * tiles * 2 * R * 4) + al((E + 1) * 4);
  b += al(64 * 8) * 4 + al((size_t)zepp_swap_decide_out_ints((int)R, (int)G, (int)nlp, 8) * 8);
  b += 9 * al(gpe * 8);
  b += 5 * al((gpe + cap / 128 + 8) * 4) + 3 * al(cap * 8) + al(cap * 4);
  b += 16 * al(R * 8) + (64 << 10);
  return b + (1 << 20);
}

template <typename T>
static int lalloc(zepp_layer* l, T** p, size_t count) {
  *p = reinterpret_cast<T*>(rt_alloc(l->rt, count * sizeof(T)));
  if (!*p) return fail("symmetric arena exhausted (need %zu more bytes)", count * sizeof(T));
  return 0;
}
#define LA(ptr, count) \
  if (lalloc(l, &(ptr), (size_t)(count))) return 1

static int layer_alloc(zepp_layer* l) {
  const int R = l->W;
  // symmetric part first: identical offsets on every rank
  for (int b = 0; b < 2; ++b) LA(l->loads_all[b], R * l->G);
  for (int b = 0; b < 2; ++b) LA(l->xchg_all[b], (size_t)R * 2 * l->SK);
  LA(l->loads_flags, R);
  LA(l->routing_flags, R);
  LA(l->x_flags, R);
  LA(l->done_flags, R);
  for (int b = 0; b < 2; ++b) LA(l->xsym[b], (size_t)l->S * l->H);
  LA(l->panel, (size_t)l->SK * l->H);
  LA(l->push_flags, R);
  if (l->cfg.swap) {
    LA(l->w1_slots, (size_t)(l->gpe + kSwapCap) * l->ffn1 * l->H);
    LA(l->w2_slots, (size_t)(l->gpe + kSwapCap) * l->H * l->I);
  }
  if (R > 1 && l->cfg.strategy == 0) LA(l->stage, (size_t)R * l->S * l->H);
  // local part
  LA(l->recv, (size_t)l->cap * l->H);
  LA(l->act, (size_t)l->cap * l->I);
  LA(l->staging, (size_t)l->cap * l->H);
  LA(l->topk_own, l->SK);
  LA(l->phys_own, l->SK);
  LA(l->probs_own, l->SK);
  LA(l->send_row, 2 * l->SK);
  LA(l->route_ws, zepp_route_workspace_ints(l->G, R));
  LA(l->route_stats, 4);
  LA(l->p2l, R * l->nlp);
  LA(l->l2p, l->G * R);
  LA(l->lcnts, l->G);
  LA(l->slot_of, l->G);
  LA(l->vce, (size_t)R * l->SK);
  LA(l->probs_all, (size_t)R * l->SK);
  LA(l->scatter_index, (size_t)R * l->SK);
  LA(l->splits, l->E_virt);
  LA(l->sps, R * l->E_virt);
  LA(l->uc, R * (R + l->NN));
  LA(l->tile_hist, (size_t)R * l->tiles_per_src * l->E_virt);
  LA(l->tile_uc, (size_t)R * l->tiles_per_src * (R + l->NN));
  LA(l->expert_base, l->E_virt + 1);
  LA(l->demands, 8);
  LA(l->dplan, zepp_dispatch_plan_words(l->L, l->NN));
  LA(l->cplan, 4 * R + 2);
  LA(l->swap_block, zepp_swap_decide_out_ints(R, l->G, l->nlp, 8));
  LA(l->gate, 2 * l->gpe);
  LA(l->sched, l->gpe);
  LA(l->redirect, l->gpe);
  LA(l->ovr0, l->gpe);
  LA(l->ovr1, l->gpe);
  LA(l->stag, 16);
  LA(l->n_tiles, 4);
  LA(l->tile_group, l->max_tiles);
  LA(l->tile_row0, l->max_tiles);
  LA(l->tile_rows, l->max_tiles);
  LA(l->tile_ready, l->max_tiles);
  LA(l->m_this, 4);
  LA(l->row_tok, l->cap);
  LA(l->row_dst, l->cap);
  LA(l->row_scale, l->cap);
  LA(l->counters, 16);
  LA(l->status, ST_WORDS);
  LA(l->step_ctr, 2);
  for (int b = 0; b < 2; ++b) LA(l->x_ptrs[b], R);
  LA(l->stage_ptrs, R);
  if (l->cfg.swap) {
    LA(l->w_ready, 2 * kSwapCap);
    LA(l->w1_peers, R);
    LA(l->w2_peers, R);
  }
  LA(l->panels, R);
  LA(l->done_ptrs, R);
  return 0;
}

extern "C" int zepp_layer_create(zepp_rt* rt, const zepp_layer_cfg* c, zepp_layer** out) {
  if (!rt->peers_ready) return fail("layer_create: peers are not mapped yet (open_peers / link_local first)");
  if (c->ranks != rt->world) return fail("layer_create: cfg.ranks %d != runtime world %d", c->ranks, rt->world);
  if (c->num_experts % c->ranks) return fail("num_experts must divide by ranks");
  if (c->ranks % c->ranks_per_node) return fail("ranks must divide by ranks_per_node");
  if (c->hidden % 128 || c->ffn_hidden % 128) return fail("hidden and ffn_hidden must be multiples of 128 (got %d, %d)", c->hidden, c->ffn_hidden);
  if (c->topk < 1 || c->topk > 64) return fail("topk out of range");
  if (c->caps[0] < 1) return fail("recv_cap must be positive");
  CU_OK(cudaSetDevice(rt->device));
  zepp_layer* l = new (std::nothrow) zepp_layer();
  if (!l) return fail("out of host memory");
  l->rt = rt;
  l->cfg = *c;
  l->G = c->num_experts; l->K = c->topk; l->H = c->hidden; l->I = c->ffn_hidden;
  l->ffn1 = c->act == 1 ? 2 * l->I : l->I;
  l->W = c->ranks; l->L = c->ranks_per_node; l->NN = l->W / l->L; l->S = c->max_tokens_per_rank;
  l->S_max = l->S;
  l->SK = l->S * l->K;
  l->nlp = l->G / l->W + c->redundant_slots_per_rank;
  l->gpe = l->nlp + 1;
  l->E_virt = l->W * l->gpe;
  l->cap = (int)c->caps[0];
  l->max_tiles = l->gpe + l->cap / kTileRowsMax + 2;
  l->tokens_per_tile = kMetaThreads / l->K;
  l->tiles_per_src = (l->S + l->tokens_per_tile - 1) / l->tokens_per_tile;
  if (l->E_virt > 4 * kMetaThreads) { delete l; return fail("too many virtual experts (%d)", l->E_virt); }
  if (l->max_tiles > kMaxTilesSmem) { delete l; return fail("recv_cap %d needs more than %d token tiles", l->cap, kMaxTilesSmem); }
  if (layer_alloc(l)) { delete l; return 1; }
  // peer tables
  const int R = l->W;
  std::vector<const __nv_bfloat16*> xp(R);
  std::vector<__nv_bfloat16*> pp(R);
  std::vector<unsigned long long*> dp(R);
  for (int b = 0; b < 2; ++b) {
    for (int p = 0; p < R; ++p) {
      l->loads_dst[b].ptr[p] = peer_ptr(rt, p, l->loads_all[b]);
      l->xchg_dst[b].ptr[p] = peer_ptr(rt, p, l->xchg_all[b]);
      xp[p] = peer_ptr(rt, p, l->xsym[b]);
    }
    CU_OK(cudaMemcpy(l->x_ptrs[b], xp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
  }
  for (int p = 0; p < R; ++p) {
    l->loads_flag_dst.ptr[p] = peer_ptr(rt, p, l->loads_flags);
    l->routing_flag_dst.ptr[p] = peer_ptr(rt, p, l->routing_flags);
    l->x_flag_dst.ptr[p] = peer_ptr(rt, p, l->x_flags);
    l->push_flag_dst.ptr[p] = peer_ptr(rt, p, l->push_flags);
    l->stage_dst.ptr[p] = l->stage ? (void*)peer_ptr(rt, p, l->stage) : nullptr;
    pp[p] = peer_ptr(rt, p, l->panel);
    dp[p] = peer_ptr(rt, p, l->done_flags);
  }
  if (l->cfg.swap) {
    std::vector<const uint4*> wp(R);
    for (int p = 0; p < R; ++p) wp[p] = (const uint4*)peer_ptr(rt, p, l->w1_slots);
    CU_OK(cudaMemcpy(l->w1_peers, wp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
    for (int p = 0; p < R; ++p) wp[p] = (const uint4*)peer_ptr(rt, p, l->w2_slots);
    CU_OK(cudaMemcpy(l->w2_peers, wp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
  }
  if (l->stage) {
    for (int p = 0; p < R; ++p) xp[p] = l->stage + (size_t)p * l->S * l->H;
    CU_OK(cudaMemcpy(l->stage_ptrs, xp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
  }
  CU_OK(cudaMemcpy(l->panels, pp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
  CU_OK(cudaMemcpy(l->done_ptrs, dp.data(), R * sizeof(void*), cudaMemcpyHostToDevice));
  const uint32_t boxes[3] = {32, 64, 128};
  for (int b = 0; b < 3; ++b) {
    if (make_map(&l->tm_recv[b], l->recv, l->cap, l->H, boxes[b])) { delete l; return 1; }
    if (make_map(&l->tm_act[b], l->act, l->cap, l->I, boxes[b])) { delete l; return 1; }
  }
  CU_OK(cudaFuncSetAttribute(moe_gemm_kernel<MODE_GATE_UP_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmCfg<MODE_GATE_UP_SWIGLU>::kSmemBytes));
  CU_OK(cudaFuncSetAttribute(moe_gemm_kernel<MODE_SINGLE_GELU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmCfg<MODE_SINGLE_GELU>::kSmemBytes));
  CU_OK(cudaFuncSetAttribute(moe_gemm_kernel<MODE_DOWN_COMBINE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmCfg<MODE_DOWN_COMBINE>::kSmemBytes));
  CU_OK(cudaFuncSetAttribute(moe_gemm_kernel<MODE_DOWN_COMBINE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmCfg<MODE_DOWN_COMBINE>::kSmemBytes));
  if (pass2_prepare(pass2_smem(l->tokens_per_tile, l->K, l->E_virt))) { delete l; return 1; }
  if (meta_fused_prepare(l)) { delete l; return 1; }
  if (l->cfg.swap && swap_decide_prepare()) { delete l; return 1; }
  {
    // CTA-pair GEMMs: attributes, resident cluster count, and whether this layer's row counts want them
    const char* pm = getenv("ZEPP_B200_PAIRS");
    if (pm != nullptr && (pm[0] == '0' || pm[0] == '1')) l->pairs_mode = pm[0] - '0';
    if (l->cfg.act == 1 && pair_kernels_prepare(l)) { delete l; return 1; }
    choose_gemm_kind(l);
    if (getenv("ZEPP_B200_VERBOSE") != nullptr)
      fprintf(stderr, "[zepp_b200] layer rank %d/%d: GEMMs on %s (pair grid %d), metadata %s, front blocks %d\n", rt->rank,
              l->W, l->use_pairs ? "CTA pairs" : "single CTAs", l->pair_grid, l->meta_fused ? "fused" : "two launches",
              l->front_blocks_max);
    const char* g = getenv("ZEPP_B200_GRAPHS");     // "0": launch the step's kernels one by one instead of as a graph
    if (g != nullptr && g[0] == '0') l->use_graphs = false;
    // The combine GEMM's epilogue stages rows in shared memory and stores whole 128-byte lines when its rows go
    // to panels on other ranks; "1" / "0" force that form on / off.
    const char* cs = getenv("ZEPP_B200_COMBINE_STAGED");
    l->combine_lines = l->W > 1;
    if (cs != nullptr && (cs[0] == '0' || cs[0] == '1')) l->combine_lines = cs[0] == '1';
  }
  if (meta_smem(l->W, l->NN, l->E_virt) > 48 * 1024) { delete l; return fail("too many ranks / experts for the metadata kernels"); }
  *out = l;
  return 0;
}

extern "C" int zepp_layer_destroy(zepp_layer* l) {
  if (l) {
    cudaSetDevice(l->rt->device);
    cudaDeviceSynchronize();
    for (auto& gph : l->graphs) cudaGraphExecDestroy(gph.exec);
    if (l->capture_stream) cudaStreamDestroy(l->capture_stream);
    delete l;
  }
  return 0;
}

extern "C" int zepp_layer_set_placement(zepp_layer* l, const int32_t* p2l, const int32_t* l2p, const int32_t* lcnts,
                                        void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  CU_OK(cudaMemcpyAsync(l->p2l, p2l, (size_t)l->W * l->nlp * 4, cudaMemcpyHostToDevice, st));
  CU_OK(cudaMemcpyAsync(l->l2p, l2p, (size_t)l->G * l->W * 4, cudaMemcpyHostToDevice, st));
  CU_OK(cudaMemcpyAsync(l->lcnts, lcnts, (size_t)l->G * 4, cudaMemcpyHostToDevice, st));
  slot_table_kernel<<<(l->G + 127) / 128, 128, 0, st>>>(l->l2p, l->lcnts, l->G, l->W, l->slot_of);
  CU_OK(cudaGetLastError());
  CU_OK(cudaStreamSynchronize(st));
  l->c_max = 1;
  for (int g = 0; g < l->G; ++g) l->c_max = lcnts[g] > l->c_max ? lcnts[g] : l->c_max;
  for (auto& gph : l->graphs) cudaGraphExecDestroy(gph.exec);     // launch sequence may change with c_max
  l->graphs.clear();
  l->have_placement = true;
  return 0;
}

extern "C" int zepp_layer_set_tokens(zepp_layer* l, int tokens) {
  if (tokens < 1 || tokens > l->S_max) return fail("set_tokens: %d is outside 1..%d (max_tokens_per_rank)", tokens, l->S_max);
  CU_OK(cudaSetDevice(l->rt->device));
  l->S = tokens;
  l->SK = tokens * l->K;
  l->tiles_per_src = (tokens + l->tokens_per_tile - 1) / l->tokens_per_tile;
  choose_gemm_kind(l);
  return meta_fused_prepare(l);
}

extern "C" int zepp_layer_weight_slots(zepp_layer* l, void** w1, void** w2) {
  if (!l->cfg.swap) return fail("weight_slots: the layer owns weight slots only with swap on");
  *w1 = l->w1_slots;
  *w2 = l->w2_slots;
  return 0;
}

extern "C" int zepp_layer_set_weights(zepp_layer* l, const void* w1, const void* w2) {
  if (l->cfg.swap) {
    // swapped experts travel between ranks: the weights live in the layer's peer-visible slots
    CU_OK(cudaSetDevice(l->rt->device));
    if (w1 != l->w1_slots) CU_OK(cudaMemcpy(l->w1_slots, w1, (size_t)l->gpe * l->ffn1 * l->H * 2, cudaMemcpyDeviceToDevice));
    if (w2 != l->w2_slots) CU_OK(cudaMemcpy(l->w2_slots, w2, (size_t)l->gpe * l->H * l->I * 2, cudaMemcpyDeviceToDevice));
    w1 = l->w1_slots;
    w2 = l->w2_slots;
  }
  const uint64_t groups = l->gpe + (l->cfg.swap ? kSwapCap : 0);       // the staging groups follow the slots
  if (make_map(&l->tm_w1, w1, groups * l->ffn1, l->H, 128)) return 1;
  if (make_map(&l->tm_w2, w2, groups * l->H, l->I, 128)) return 1;
  for (auto& gph : l->graphs) cudaGraphExecDestroy(gph.exec);     // the tensor maps are baked into captured launches
  l->graphs.clear();
  l->have_weights = true;
  return 0;
}

#define LAUNCH_OK()                                                                          \
  do {                                                                                       \
    cudaError_t _e = cudaGetLastError();                                                     \
    if (_e != cudaSuccess) return fail("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
    l->launches++;                                                                           \
  } while (0)

static bool needs_loads(const zepp_layer* l);
// One rank, one replica per expert, nobody consuming the loads: the routing is a slot lookup that the
// first metadata kernel does itself (no routing launch).
static bool local_route(const zepp_layer* l) { return l->W == 1 && l->c_max <= 1 && !needs_loads(l) && !l->cfg.swap; }

static MetaArgs layer_meta_args(zepp_layer* l) {
  MetaArgs m{};
  m.gathered = l->xchg_all[0];
  m.gathered_odd = l->xchg_all[1];
  m.vce_in = nullptr;
  m.R = l->W; m.L = l->L; m.S = l->S; m.K = l->K; m.nlp = l->nlp; m.gpe = l->gpe; m.my_rank = l->rt->rank;
  m.tokens_per_tile = l->tokens_per_tile; m.tiles_per_src = l->tiles_per_src;
  m.vce = l->vce; m.probs_all = l->probs_all; m.splits = l->splits; m.scatter_index = l->scatter_index;
  m.sps = l->sps; m.uc = l->uc; m.demands = l->demands;
  for (int i = 0; i < 8; ++i) m.caps[i] = l->cfg.caps[i];
  m.direct = l->cfg.strategy == 1; m.relay_slots = 2;
  m.dplan = nullptr; m.cplan = nullptr; m.copies_per_rank = l->SK;     // plan heads: on request (zepp_layer_table)
  m.tile_hist = l->tile_hist; m.tile_uc = l->tile_uc; m.expert_base = l->expert_base;
  m.n_tiles = l->n_tiles; m.tile_group = l->tile_group; m.tile_row0 = l->tile_row0; m.tile_rows = l->tile_rows;
  m.tile_ready = l->tile_ready; m.max_tiles = l->max_tiles; m.recv_cap = l->cap; m.m_this = l->m_this;
  m.row_tok = l->row_tok; m.row_dst = l->row_dst; m.row_scale = l->row_scale; m.hidden = l->H;
  m.tile_rows_max = l->use_pairs ? kPairTileRows : kTileRowsMax;
  m.group_order = l->cfg.swap ? l->sched : nullptr;
  m.group_redirect = l->cfg.swap ? l->redirect : nullptr;
  m.staged = l->stage != nullptr ? 1 : 0;
  m.routing_flags = l->W > 1 ? l->routing_flags : nullptr;
  m.epoch_ptr = l->step_ctr; m.limit_ns = l->rt->wait_ns; m.status = l->status;
  m.block_counter = l->counters + 8;
  m.grid_sync = l->counters + 14;
  if (local_route(l)) {
    m.local_topk = l->ids_in; m.local_probs = l->wts_in; m.slot_of = l->slot_of; m.G = l->G;
    m.phys_own = l->phys_own; m.send_row = l->send_row;
    m.gathered_out = l->xchg_all[0]; m.gathered_out_odd = l->xchg_all[1]; m.ctr = l->step_ctr;
  }
  return m;
}

static size_t meta_smem(int R, int NN, int E_virt) {
  const size_t a = (size_t)(E_virt + R + NN), b = meta_scan_smem_ints(R, NN, E_virt);   // pass1 counters / the scan
  return (a > b ? a : b) * sizeof(int);
}
static size_t fused_smem(const zepp_layer* l) {
  return meta_fused_smem_ints(l->W, l->NN, l->E_virt, l->tokens_per_tile, l->K) * sizeof(int);
}
// CTA pairs pay once experts have several hundred rows each (measured: +7 % on the dispatch GEMM at 512 rows per expert
// on one GPU, nothing at 256 rows per expert across 8 GPUs, and a loss where a step is bound by streaming the weights
// from HBM, because a pair keeps fewer weight bytes in flight per SM than two single CTAs).
static void choose_gemm_kind(zepp_layer* l) {
  const long long rows_per_expert = (long long)l->S * l->K * l->W / (l->G > 0 ? l->G : 1);
  bool pairs = l->cfg.act == 1 && l->pair_grid >= 2 && rows_per_expert >= 384;
  if (l->pairs_mode == 0) pairs = false;
  if (l->pairs_mode == 1) pairs = l->cfg.act == 1 && l->pair_grid >= 2;
  if (pairs != l->use_pairs) {
    for (auto& gph : l->graphs) cudaGraphExecDestroy(gph.exec);
    l->graphs.clear();
  }
  l->use_pairs = pairs;
}

// Push blocks a front launch can add beside its metadata and route blocks (0: the push stays a kernel of its own).
static int front_push_blocks(const zepp_layer* l, int n_route) {
  int n = l->front_blocks_max - (l->W * l->tiles_per_src + 1) - n_route;
  if (n > 128) n = 128;
  if (n < 1 || (l->S + n - 1) / n > kPushMaxTokensPerBlock) return 0;
  return n;
}
// Can the metadata of the current bucket run as one cooperative launch (every block resident at once)?
static int meta_fused_prepare(zepp_layer* l) {
  l->meta_fused = false;
  const size_t bytes = fused_smem(l);
  if (bytes > 200 * 1024) return 0;
  const char* off = getenv("ZEPP_B200_META_FUSED");
  if (off != nullptr && off[0] == '0') return 0;
  if (bytes > 48 * 1024)
    CU_OK(cudaFuncSetAttribute(meta_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  int per_sm = 0;
  CU_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, meta_fused_kernel, kMetaThreads, bytes));
  l->front_blocks_max = per_sm * l->rt->sm_count;
  l->meta_fused = l->front_blocks_max >= l->W * l->tiles_per_src + 1;
  return 0;
}
static size_t pass2_smem(int tokens_per_tile, int K, int E_virt) {
  return (size_t)((tokens_per_tile * K + 31) / 32) * E_virt * sizeof(int);
}
// Kernel attributes belong to a device's instance of a function: remembered per device ordinal.
constexpr int kMaxDevices = 64;
static std::mutex g_attr_mutex;
static size_t g_pass2_granted[kMaxDevices] = {};
static bool g_swap_attr[kMaxDevices] = {};

// ZEPP_B200_VACATE_STAGED=0 keeps the vacate pass's budget tables in global memory even when they would fit in
// shared memory (the form large expert counts take), so that tests reach it on small cases.
static bool vacate_tables_in_global() {
  const char* e = getenv("ZEPP_B200_VACATE_STAGED");
  return e != nullptr && e[0] == '0';
}

static int pass2_prepare(size_t bytes) {
  if (bytes > 200 * 1024) return fail("metadata: %zu bytes of shared memory per tile exceed the SM", bytes);
  if (bytes <= 48 * 1024) return 0;
  int dev = -1;
  CU_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  if (dev < 0 || dev >= kMaxDevices || bytes > g_pass2_granted[dev]) {
    CU_OK(cudaFuncSetAttribute(meta_pass2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (dev >= 0 && dev < kMaxDevices) g_pass2_granted[dev] = bytes;
  }
  return 0;
}

// Does this step need the gathered loads?  Only the water-fill (some expert has more than one
// replica) and the swap decision consume them.
static bool needs_loads(const zepp_layer* l) { return l->c_max > 1 || l->cfg.swap != 0; }

static SimpleRouteArgs layer_simple_route_args(zepp_layer* l) {
  SimpleRouteArgs sa{};
  const int R = l->W;
  sa.topk_own = l->ids_in; sa.probs_own = l->wts_in; sa.slot_of = l->slot_of;
  sa.SK = l->SK; sa.G = l->G; sa.R = R; sa.my_rank = l->rt->rank; sa.world = R; sa.first = needs_loads(l) ? 0 : 1;
  sa.phys_own = l->phys_own; sa.send_row = l->send_row; sa.dst = l->xchg_dst[0]; sa.dst_odd = l->xchg_dst[1];
  sa.flags = l->routing_flag_dst; sa.ctr = l->step_ctr; sa.block_counter = l->counters + 0; sa.status = l->status;
  return sa;
}

static PushArgs layer_push_args(zepp_layer* l, const void* x) {
  PushArgs pa{};
  pa.phys_own = l->phys_own; pa.x = (const __nv_bfloat16*)x; pa.stage = l->stage_dst; pa.flags = l->push_flag_dst;
  pa.S = l->S; pa.K = l->K; pa.H = l->H; pa.nlp = l->nlp; pa.rank = l->rt->rank; pa.world = l->W;
  pa.region_tokens = l->S_max; pa.G = l->G;
  pa.epoch_ptr = l->step_ctr; pa.counter = l->counters + 10; pa.status = l->status;
  return pa;
}

extern "C" int zepp_layer_prepare_phase(zepp_layer* l, int phase, const int32_t* ids, const float* wts, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  CU_OK(cudaSetDevice(l->rt->device));
  if (!l->have_placement) return fail("prepare: no placement set");
  const int R = l->W, me = l->rt->rank;
  if (phase == 0) {
    l->epoch += 1;                 // host mirror of the device step counter
    // the routing inputs are read in place by this step's kernels (stream order keeps them valid)
    l->ids_in = ids;
    l->wts_in = wts;
    if (needs_loads(l)) {
      loads_publish_kernel<<<1, 1024, l->G * sizeof(int), st>>>(ids, l->SK, l->G, me, R, l->loads_dst[0], l->loads_dst[1],
                                                               l->loads_flag_dst, l->step_ctr, l->status, l->route_stats);
      LAUNCH_OK();
    }
    return 0;
  }
  if (phase == 1) {
    if (!l->cfg.swap) return 0;
    // swap: one launch waits for the gathered loads, decides (rewrites p2l / l2p on the device), rebuilds the
    // router's slot table and marks this rank's incoming slots.  The weights move under the GEMMs.  Nothing is
    // read on the host.
    SwapArgs sa = swap_args(l->loads_all[0], l->p2l, l->l2p, l->lcnts, R, l->G, l->L, l->nlp,
                            (double)l->cfg.c_num / (double)l->cfg.c_den, 8, 32, l->swap_block);
    sa.loads_odd = l->loads_all[1]; sa.epoch_ptr = l->step_ctr; sa.loads_flags = R > 1 ? l->loads_flags : nullptr;
    sa.limit_ns = l->rt->wait_ns; sa.status = l->status; sa.slot_of = l->slot_of; sa.rank = me;
    sa.sched = l->sched; sa.redirect = l->redirect; sa.ready = l->w_ready;
    swap_decide_kernel<<<1, kSwapThreads, swap_smem(R, l->G, l->L, l->nlp), st>>>(sa);
    LAUNCH_OK();
    return 0;
  }
  if (phase == 2) {
    if (ids) { l->ids_in = ids; l->wts_in = wts; }
    if (local_route(l)) return 0;        // done by the first metadata kernel
    if (l->c_max <= 1 && l->front_route) return 0;      // the front kernel's route blocks do it
    if (l->c_max <= 1) {
      SimpleRouteArgs sa = layer_simple_route_args(l);
      sa.route_blocks = (l->SK / 4 + 255) / 256 > 0 ? (l->SK / 4 + 255) / 256 : 1;
      if ((l->SK & 3) != 0) sa.route_blocks = (l->SK + 255) / 256;
      int grid = sa.route_blocks;
      if (l->fuse_x != nullptr && R > 1) {
        // the caller's x is already known (zepp_layer_step): publish it from extra blocks of this launch
        sa.x = (const uint4*)l->fuse_x; sa.xsym_even = (uint4*)l->xsym[0]; sa.xsym_odd = (uint4*)l->xsym[1];
        sa.x_vec = (size_t)l->S * l->H / 8; sa.x_flags = l->x_flag_dst;
        grid += 64;
        l->x_fused = l->fuse_x;
      }
      route_simple_publish_kernel<<<grid, 256, l->G * sizeof(int), st>>>(sa);
      LAUNCH_OK();
    } else {
      RouteArgs ra{};
      ra.topk_own = l->ids_in; ra.n_entries = l->SK; ra.loads = l->loads_all[0]; ra.loads_odd = l->loads_all[1];
      ra.l2p = l->l2p; ra.lcnts = l->lcnts;
      ra.G = l->G; ra.R = R; ra.L = l->L; ra.nlp = l->nlp; ra.my_rank = me;
      ra.c_num = l->cfg.c_num; ra.c_den = l->cfg.c_den; ra.ws = l->route_ws; ra.phys_own = l->phys_own;
      ra.loads_flags = R > 1 ? l->loads_flags : nullptr;
      ra.epoch_ptr = l->step_ctr; ra.limit_ns = l->rt->wait_ns; ra.status = l->status; ra.stats = l->route_stats;
      route_kernel<<<(l->G + 7) / 8, 256, 0, st>>>(ra);
      LAUNCH_OK();
      FinishArgs fa{};
      fa.topk_own = l->ids_in; fa.phys_own = l->phys_own; fa.probs_own = l->wts_in;
      fa.S = l->S; fa.K = l->K; fa.G = l->G; fa.R = R; fa.L = l->L; fa.nlp = l->nlp; fa.my_rank = me;
      fa.ws = l->route_ws; fa.send_row = l->send_row; fa.dst = l->xchg_dst[0]; fa.dst_odd = l->xchg_dst[1];
      fa.flags = l->routing_flag_dst;
      fa.world = R; fa.epoch_ptr = l->step_ctr; fa.block_counter = l->counters + 0; fa.status = l->status;
      fa.stats = l->route_stats;
      if (l->NN > 1) {
        const VacateShape vs = vacate_shape(l->G, R, l->K, l->nlp, vacate_tables_in_global());
        route_vacate_kernel<<<1, kVacWarps * 32, vs.smem, st>>>(fa, vs.staged, vs.chunk);
        LAUNCH_OK();
      }
      route_finish_kernel<<<8, 256, 0, st>>>(fa);
      LAUNCH_OK();
    }
    return 0;
  }
  if (phase == 3) {
    MetaArgs m = layer_meta_args(l);
    const int grid = R * l->tiles_per_src;
    if (l->meta_fused) {
      FrontArgs f{};
      if (l->front_route) {
        f.route = layer_simple_route_args(l);
        f.n_route = ((l->SK + 3) / 4 + kMetaThreads - 1) / kMetaThreads;
        f.first = f.route.first;
        f.route_counter = l->counters + 0;
      }
      if (l->front_push) {
        f.push = layer_push_args(l, l->fuse_x);
        if (l->front_route) { f.push.phys_own = nullptr; f.push.topk_own = l->ids_in; f.push.slot_of = l->slot_of; }
        f.n_push = front_push_blocks(l, f.n_route);
      }
      void* args[] = {(void*)&m, (void*)&f};
      CU_OK(cudaLaunchCooperativeKernel((const void*)meta_fused_kernel, dim3(grid + 1 + f.n_route + f.n_push),
                                        dim3(kMetaThreads), args, fused_smem(l), st));
      l->launches++;
      return 0;
    }
    meta_pass1_kernel<<<grid, kMetaThreads, meta_smem(R, l->NN, l->E_virt), st>>>(m);      // + scan in its last block
    LAUNCH_OK();
    meta_pass2_kernel<<<grid, kMetaThreads, pass2_smem(l->tokens_per_tile, l->K, l->E_virt), st>>>(m);
    LAUNCH_OK();
    return 0;
  }
  return fail("prepare: bad phase %d", phase);
}

extern "C" int zepp_layer_prepare(zepp_layer* l, const int32_t* ids, const float* wts, void* stream) {
  for (int ph = 0; ph < 4; ++ph)
    if (zepp_layer_prepare_phase(l, ph, ids, wts, stream)) return 1;
  return 0;
}

static GemmArgs layer_gemm_args(zepp_layer* l, bool first) {
  GemmArgs g{};
  g.tt.n_tiles = l->n_tiles; g.tt.tile_group = l->tile_group; g.tt.tile_row0 = l->tile_row0; g.tt.tile_rows = l->tile_rows;
  g.k_extent = first ? l->H : l->I;
  // dispatch GEMM: one 128-feature block of gate and of up per item (or of W1 alone without a gate);
  // combine GEMM: two neighbouring 128-feature blocks of W2 per item
  g.n_feat_tiles = first ? l->I / kTileM : (l->H + 2 * kTileM - 1) / (2 * kTileM);
  g.w_rows_per_group = first ? l->ffn1 : l->H;
  g.up_row_offset = first ? l->I : kTileM;
  g.act = l->act; g.ld_act = l->I;
  g.row_scale = l->row_scale; g.row_dst = l->row_dst; g.panels = l->panels; g.staging = nullptr;
  g.done_flags = nullptr; g.cta_counter = l->counters + 2;
  g.world = l->W; g.rank = l->rt->rank; g.epoch_ptr = l->step_ctr;
  g.row_tok = l->row_tok; g.x_ptrs = l->x_ptrs[0]; g.x_ptrs_odd = l->x_ptrs[1];
  g.x_self = (const __nv_bfloat16*)l->x_self;
  g.x_flags = l->W > 1 ? l->x_flags : nullptr;
  if (l->stage != nullptr) {       // staged dispatch: rows were pushed into this rank's staging regions
    g.x_ptrs = l->stage_ptrs; g.x_ptrs_odd = l->stage_ptrs; g.x_self = nullptr; g.x_flags = l->push_flags;
  }
  g.recv = l->recv; g.tile_ready = l->tile_ready; g.tokens_per_rank = l->S; g.gather = 0;
  if (l->cfg.swap) {
    g.swap_block = l->swap_block; g.swap_ranks = l->W; g.swap_cap = kSwapCap; g.n_groups = l->gpe;
    g.w_peers = first ? l->w1_peers : l->w2_peers;
    g.w_slots = (uint4*)(first ? l->w1_slots : l->w2_slots);
    g.w_vec = (unsigned long long)(first ? (size_t)l->ffn1 * l->H : (size_t)l->H * l->I) / 8;
    g.w_ready = l->w_ready + (first ? 0 : kSwapCap);
  }
  g.status = l->status; g.mbar_limit_ns = 2 * l->rt->wait_ns + 1000000000ull; g.flag_limit_ns = l->rt->wait_ns;
  return g;
}

template <int MODE, bool LINES = false>
static int launch_gemm(zepp_layer* l, const CUtensorMap& tw, const CUtensorMap* tx, GemmArgs& g, cudaStream_t st) {
  // more gather warps when most rows cross NVLink (latency-bound pulls), fewer when they are local
  const bool movers = g.swap_block != nullptr && l->W > 1;
  if (!movers) g.swap_block = nullptr;
  const int threads = g.gather ? 192 + 32 * (l->W >= 4 ? kMaxGatherWarps : 4) : (movers ? 192 + 32 * 4 : 192);
  const bool coop = g.gather || movers;     // spare warps of one CTA feed the producers of others: every CTA must be resident
  void* args[] = {(void*)&tw, (void*)&tx[0], (void*)&tx[1], (void*)&tx[2], (void*)&g};
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.blockDim = dim3(threads);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = coop ? 1 : 0;
  if constexpr (MODE != MODE_SINGLE_GELU) {
    if (l->use_pairs) {
      cfg.gridDim = dim3(l->pair_grid);
      cfg.dynamicSmemBytes = kPairSmemBytes;
      CU_OK(cudaLaunchKernelExC(&cfg, (const void*)moe_gemm_pair_kernel<MODE, LINES>, args));
      l->launches++;
      return 0;
    }
  }
  cfg.gridDim = dim3(l->rt->sm_count);
  cfg.dynamicSmemBytes = GemmCfg<MODE>::kSmemBytes;
  CU_OK(cudaLaunchKernelExC(&cfg, (const void*)moe_gemm_kernel<MODE, LINES>, args));
  l->launches++;
  return 0;
}

// Attributes of the CTA-pair kernels and how many pairs the device keeps resident (one CTA per SM).
static int pair_kernels_prepare(zepp_layer* l) {
  CU_OK(cudaFuncSetAttribute(moe_gemm_pair_kernel<MODE_GATE_UP_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
  CU_OK(cudaFuncSetAttribute(moe_gemm_pair_kernel<MODE_DOWN_COMBINE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
  CU_OK(cudaFuncSetAttribute(moe_gemm_pair_kernel<MODE_DOWN_COMBINE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(l->rt->sm_count & ~1);
  cfg.blockDim = dim3(192 + 32 * kMaxGatherWarps);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  int clusters = 0;
  cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, (const void*)moe_gemm_pair_kernel<MODE_DOWN_COMBINE, true>, &cfg);
  if (e != cudaSuccess) { cudaGetLastError(); clusters = 0; }
  if (clusters > l->rt->sm_count / 2) clusters = l->rt->sm_count / 2;
  l->pair_grid = 2 * clusters;
  return 0;
}

static SwapCommitArgs layer_commit_args(zepp_layer* l) {
  SwapCommitArgs c{};
  if (!l->cfg.swap || l->W == 1) return c;
  c.block = l->swap_block; c.R = l->W; c.rank = l->rt->rank; c.cap = kSwapCap; c.gpe = l->gpe;
  c.w1_vec = (size_t)l->ffn1 * l->H / 8; c.w2_vec = (size_t)l->H * l->I / 8;
  c.w1 = (uint4*)l->w1_slots; c.w2 = (uint4*)l->w2_slots;
  return c;
}

static MoveArgs layer_move_args(zepp_layer* l) {
  MoveArgs m{};
  m.m_this = l->m_this; m.row_tok = l->row_tok; m.row_dst = l->row_dst;
  m.x_ptrs = l->x_ptrs[0]; m.x_ptrs_odd = l->x_ptrs[1]; m.x_self = (const __nv_bfloat16*)l->x_self;
  m.recv = l->recv; m.staging = l->staging; m.panels = l->panels; m.done_flags = l->done_ptrs;
  m.x_flags = l->W > 1 ? l->x_flags : nullptr; m.counter = l->counters + 4;
  m.H = l->H; m.S = l->S; m.world = l->W; m.rank = l->rt->rank; m.recv_cap = l->cap;
  m.epoch_ptr = l->step_ctr; m.limit_ns = l->rt->wait_ns; m.status = l->status;
  return m;
}

extern "C" int zepp_layer_forward_phase(zepp_layer* l, int phase, const void* x, void* y, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  CU_OK(cudaSetDevice(l->rt->device));
  if (!l->have_weights) return fail("forward: no weights set");
  if (l->epoch == 0) return fail("forward: prepare has not run");
  const bool direct = l->cfg.strategy == 1;
  if (phase == 0) {
    l->x_self = x;
    if (l->x_fused == x && x != nullptr) {     // already published by the routing kernel of this step
      l->x_fused = nullptr;
      return 0;
    }
    if (l->stage != nullptr) {
      if (l->front_push) return 0;               // pushed by the front kernel of this step
      PushArgs pa = layer_push_args(l, x);
      int grid = 2 * l->rt->sm_count;
      if (grid > l->S) grid = l->S;
      if (grid * 64 < l->S) grid = (l->S + 63) / 64;
      dispatch_push_kernel<<<grid, 256, 0, st>>>(pa);
      LAUNCH_OK();
      return 0;
    }
    if (l->W > 1) {
      const size_t n_vec = (size_t)l->S * l->H / 8;
      publish_x_kernel<<<64, 256, 0, st>>>((const uint4*)x, (uint4*)l->xsym[0], (uint4*)l->xsym[1], n_vec, l->rt->rank,
                                          l->W, l->x_flag_dst, l->step_ctr, l->counters + 6);
      LAUNCH_OK();
    }
    return 0;
  }
  if (phase == 1) {
    l->x_self = x;
    GemmArgs g = layer_gemm_args(l, true);
    if (direct) {
      MoveArgs m = layer_move_args(l);
      dispatch_pull_kernel<<<l->rt->sm_count * 2, 256, 0, st>>>(m);
      LAUNCH_OK();
    } else {
      g.gather = 1;
    }
    if (l->cfg.act == 1) return launch_gemm<MODE_GATE_UP_SWIGLU>(l, l->tm_w1, l->tm_recv, g, st);
    return launch_gemm<MODE_SINGLE_GELU>(l, l->tm_w1, l->tm_recv, g, st);
  }
  if (phase == 2) {
    GemmArgs g = layer_gemm_args(l, false);
    if (direct) {
      g.staging = l->staging;
    } else if (l->W > 1) {
      g.done_flags = l->done_ptrs;
    }
    if (l->combine_lines) {
      if (launch_gemm<MODE_DOWN_COMBINE, true>(l, l->tm_w2, l->tm_act, g, st)) return 1;
    } else {
      if (launch_gemm<MODE_DOWN_COMBINE>(l, l->tm_w2, l->tm_act, g, st)) return 1;
    }
    if (direct) {
      MoveArgs m = layer_move_args(l);
      combine_push_kernel<<<l->rt->sm_count * 2, 256, 0, st>>>(m);
      LAUNCH_OK();
    }
    return 0;
  }
  if (phase == 3) {
    combine_reduce_kernel<<<l->rt->sm_count * 2, 256, 0, st>>>(l->panel, (__nv_bfloat16*)y, l->S, l->K, l->H,
                                                            l->W > 1 ? l->done_flags : nullptr, l->W, l->step_ctr,
                                                            l->rt->wait_ns, l->status, layer_commit_args(l));
    LAUNCH_OK();
    return 0;
  }
  return fail("forward: bad phase %d", phase);
}

extern "C" int zepp_layer_forward(zepp_layer* l, const void* x, void* y, void* stream) {
  for (int ph = 0; ph < 4; ++ph)
    if (zepp_layer_forward_phase(l, ph, x, y, stream)) return 1;
  return 0;
}

// One whole step in launch order.  x is published right after the first planning kernel, long before
// the dispatch GEMM of any rank needs it, so the GEMM's wait for x never stalls on rank skew.
static int step_enqueue(zepp_layer* l, const int32_t* ids, const float* wts, const void* x, void* y, void* stream) {
  l->ids_in = ids;
  l->wts_in = wts;
  // roles the front kernel takes over in a whole-step call (x is known before the planning starts)
  const bool staged = l->stage != nullptr;
  const int n_route_blocks = ((l->SK + 3) / 4 + kMetaThreads - 1) / kMetaThreads;
  l->front_route = staged && l->meta_fused && l->c_max <= 1 &&
                   l->front_blocks_max >= l->W * l->tiles_per_src + 1 + n_route_blocks;
  l->front_push = staged && l->meta_fused && front_push_blocks(l, l->front_route ? n_route_blocks : 0) > 0;
  l->fuse_x = (l->front_push || (!needs_loads(l) && l->c_max <= 1 && !staged)) ? x : nullptr;
  l->x_fused = nullptr;
  int rc = 0;
  for (int ph = 0; ph < 3 && !rc; ++ph) rc = zepp_layer_prepare_phase(l, ph, ids, wts, stream);
  // unfused dispatch with a loads exchange: publish x before the metadata so that no rank's pull waits for it
  if (!rc && !staged && l->x_fused == nullptr) rc = zepp_layer_forward_phase(l, 0, x, y, stream);
  if (!rc) rc = zepp_layer_prepare_phase(l, 3, ids, wts, stream);
  if (!rc && staged) rc = zepp_layer_forward_phase(l, 0, x, y, stream);      // no-op when the front kernel pushed
  for (int ph = 1; ph < 4 && !rc; ++ph) rc = zepp_layer_forward_phase(l, ph, x, y, stream);
  l->fuse_x = nullptr;
  l->front_route = l->front_push = false;
  return rc;
}

// prepare + forward as one call.  The launch sequence of a step depends only on the four
// pointers (every count, offset and the epoch live in device memory), so it is captured once
// per pointer set into a CUDA graph and replayed: one graph launch per step instead of 6-9
// kernel launches.
extern "C" int zepp_layer_step(zepp_layer* l, const int32_t* ids, const float* wts, const void* x, void* y, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  CU_OK(cudaSetDevice(l->rt->device));
  if (!l->have_weights) return fail("step: no weights set");
  if (!l->use_graphs) return step_enqueue(l, ids, wts, x, y, stream);
  for (auto& gph : l->graphs) {
    if (gph.ids == ids && gph.wts == wts && gph.x == x && gph.y == y && gph.tokens == l->S) {
      CU_OK(cudaGraphLaunch(gph.exec, st));
      l->epoch += 1;
      l->launches += gph.kernels;
      l->x_self = x; l->ids_in = ids; l->wts_in = wts;
      return 0;
    }
  }
  if (l->graphs.size() >= 128) return step_enqueue(l, ids, wts, x, y, stream);
  const int64_t before = l->launches;
  const unsigned long long epoch_before = l->epoch;
  cudaGraph_t graph = nullptr;
  // recorded on a stream of the layer's own (the caller's may be the legacy default stream, which
  // cannot capture); the instantiated graph is launched on the caller's stream
  if (l->capture_stream == nullptr) CU_OK(cudaStreamCreateWithFlags(&l->capture_stream, cudaStreamNonBlocking));
  if (cudaStreamBeginCapture(l->capture_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    l->use_graphs = false;
    return step_enqueue(l, ids, wts, x, y, stream);
  }
  const int rc = step_enqueue(l, ids, wts, x, y, (void*)l->capture_stream);
  cudaError_t e = cudaStreamEndCapture(l->capture_stream, &graph);
  l->epoch = epoch_before;           // nothing ran yet: the capture only recorded the launches
  const int64_t kernels = l->launches - before;
  l->launches = before;
  if (rc != 0 || e != cudaSuccess || graph == nullptr) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    l->use_graphs = false;           // fall back to plain launches for good
    return step_enqueue(l, ids, wts, x, y, stream);
  }
  zepp_layer::StepGraph gph{};
  gph.ids = ids; gph.wts = wts; gph.x = x; gph.y = y; gph.tokens = l->S; gph.kernels = kernels;
  e = cudaGraphInstantiate(&gph.exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    cudaGetLastError();
    l->use_graphs = false;
    return step_enqueue(l, ids, wts, x, y, stream);
  }
  l->graphs.push_back(gph);
  CU_OK(cudaGraphLaunch(gph.exec, st));
  l->epoch += 1;
  l->launches += kernels;
  return 0;
}

extern "C" int zepp_layer_status(zepp_layer* l, void* stream, uint64_t out[8]) {
  cudaStream_t st = (cudaStream_t)stream;
  CU_OK(cudaSetDevice(l->rt->device));
  CU_OK(cudaStreamSynchronize(st));
  CU_OK(cudaMemcpy(out, l->status, 8 * 8, cudaMemcpyDeviceToHost));
  CU_OK(cudaMemset(l->status, 0, 4 * 8));
  return 0;
}

extern "C" int zepp_layer_trace(zepp_layer* l, void* stream, uint64_t out[64]) {
  CU_OK(cudaSetDevice(l->rt->device));
  CU_OK(cudaStreamSynchronize((cudaStream_t)stream));
  CU_OK(cudaMemcpy(out, l->status, ST_WORDS * 8, cudaMemcpyDeviceToHost));
  CU_OK(cudaMemset(l->status + TR_GEMM1_END, 0, 8));
  CU_OK(cudaMemset(l->status + TR_GEMM2_END, 0, 8));
  CU_OK(cudaMemset(l->status + TR_REDUCE_END, 0, 8));
  CU_OK(cudaMemset(l->status + 30, 0, 16));
  return 0;
}

extern "C" int zepp_layer_gpu_launches(zepp_layer* l, int64_t* out) {
  *out = l->launches;
  return 0;
}

extern "C" int zepp_layer_table(zepp_layer* l, int which, void** p, size_t* bytes) {
  const size_t R = l->W, SK = l->SK;
  const int b = (int)(l->epoch & 1);
  switch (which) {
    case ZEPP_T_LOADS: *p = l->loads_all[b]; *bytes = R * l->G * 4; break;
    case ZEPP_T_PHYS_OWN: *p = l->phys_own; *bytes = SK * 4; break;
    case ZEPP_T_VCE: *p = l->vce; *bytes = R * SK * 4; break;
    case ZEPP_T_PROBS_ALL: *p = l->probs_all; *bytes = R * SK * 4; break;
    case ZEPP_T_SPLITS: *p = l->splits; *bytes = (size_t)l->E_virt * 4; break;
    case ZEPP_T_SCATTER_INDEX: *p = l->scatter_index; *bytes = R * SK * 4; break;
    case ZEPP_T_SPS: *p = l->sps; *bytes = R * l->E_virt * 4; break;
    case ZEPP_T_UC: *p = l->uc; *bytes = R * (R + l->NN) * 4; break;
    case ZEPP_T_DEMANDS: *p = l->demands; *bytes = 64; break;
    case ZEPP_T_DPLAN:
    case ZEPP_T_CPLAN: {
      // computed on request from the last step's counts; synchronises the device
      CU_OK(cudaSetDevice(l->rt->device));
      CU_OK(cudaDeviceSynchronize());
      MetaArgs m = layer_meta_args(l);
      m.dplan = l->dplan;
      m.cplan = l->NN == 1 ? l->cplan : nullptr;
      plan_heads_kernel<<<1, 128, (size_t)(l->W * l->W + l->W * (l->W + l->NN)) * sizeof(int), 0>>>(m);
      CU_OK(cudaGetLastError());
      CU_OK(cudaDeviceSynchronize());
      if (which == ZEPP_T_CPLAN) { *p = l->cplan; *bytes = (4 * R + 2) * 8; break; }
      *p = l->dplan; *bytes = (size_t)zepp_dispatch_plan_words(l->L, l->NN) * 8; break;
    }
    case ZEPP_T_ROUTE_WS: *p = l->route_ws; *bytes = (size_t)zepp_route_workspace_ints(l->G, l->W) * 4; break;
    case ZEPP_T_SWAP_BLOCK: *p = l->swap_block; *bytes = (size_t)zepp_swap_decide_out_ints(l->W, l->G, l->nlp, 8) * 8; break;
    case ZEPP_T_M_THIS: *p = l->m_this; *bytes = 8; break;
    case ZEPP_T_ROW_TOK: *p = l->row_tok; *bytes = (size_t)l->cap * 4; break;
    case ZEPP_T_ACT: *p = l->act; *bytes = (size_t)l->cap * l->I * 2; break;
    case ZEPP_T_RECV: *p = l->recv; *bytes = (size_t)l->cap * l->H * 2; break;
    case ZEPP_T_P2L: *p = l->p2l; *bytes = R * l->nlp * 4; break;
    case ZEPP_T_L2P: *p = l->l2p; *bytes = (size_t)l->G * R * 4; break;
    case ZEPP_T_N_TILES: *p = l->n_tiles; *bytes = 4; break;
    case ZEPP_T_PANEL: *p = l->panel; *bytes = SK * l->H * 2; break;
    case ZEPP_T_GATE: *p = l->gate; *bytes = (size_t)2 * l->gpe * 8; break;
    case ZEPP_T_SCHED: *p = l->sched; *bytes = (size_t)l->gpe * 4; break;
    default: return fail("layer_table: unknown table %d", which);
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// stand-alone planner entry points
// ---------------------------------------------------------------------------------------------
extern "C" int zepp_route_workspace_ints(int G, int R) { return route_ws_layout(G, R).total; }

extern "C" int zepp_route_ws_offsets(int G, int R, int64_t o[10]) {
  const RouteWs w = route_ws_layout(G, R);
  o[0] = w.rep; o[1] = w.rphys; o[2] = w.c; o[3] = w.D; o[4] = w.U; o[5] = w.Lb; o[6] = w.fill; o[7] = w.M;
  o[8] = w.rel; o[9] = w.ext;
  return 0;
}

extern "C" int zepp_route(const int32_t* topk_own, int S, int K, const int32_t* loads, const int32_t* l2p,
                          const int32_t* lcnts, int G, int R, int my_rank, int nlp, int L, int64_t c_num, int64_t c_den,
                          int32_t* ws, const float* probs_own, int32_t* send_row, int32_t* phys_own, int64_t* stats,
                          void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (R < 1 || R > kMaxRanks || L < 1 || R % L) return fail("route: bad topology R=%d L=%d", R, L);
  if (K > 64) return fail("route: topk > 64");
  RouteArgs ra{};
  ra.topk_own = topk_own; ra.n_entries = S * K; ra.loads = loads; ra.l2p = l2p; ra.lcnts = lcnts;
  ra.G = G; ra.R = R; ra.L = L; ra.nlp = nlp; ra.my_rank = my_rank; ra.c_num = c_num; ra.c_den = c_den;
  ra.ws = ws; ra.phys_own = phys_own; ra.loads_flags = nullptr; ra.epoch_ptr = nullptr; ra.limit_ns = 0; ra.status = nullptr;
  ra.stats = (long long*)stats;
  if (stats) CU_OK(cudaMemsetAsync(stats, 0, 32, st));
  route_kernel<<<(G + 7) / 8, 256, 0, st>>>(ra);
  CU_OK(cudaGetLastError());
  FinishArgs fa{};
  fa.topk_own = topk_own; fa.phys_own = phys_own; fa.probs_own = probs_own; fa.S = S; fa.K = K; fa.G = G; fa.R = R;
  fa.L = L; fa.nlp = nlp; fa.my_rank = my_rank; fa.ws = ws; fa.send_row = send_row; fa.world = 0; fa.epoch_ptr = nullptr;
  fa.status = nullptr; fa.stats = (long long*)stats;
  if (R / L > 1 && topk_own != nullptr) {
    const VacateShape vs = vacate_shape(G, R, K, nlp, vacate_tables_in_global());
    route_vacate_kernel<<<1, kVacWarps * 32, vs.smem, st>>>(fa, vs.staged, vs.chunk);
    CU_OK(cudaGetLastError());
  }
  if (send_row != nullptr && probs_own != nullptr) {
    fa.block_counter = nullptr;                  // one block: it is its own last block
    route_finish_kernel<<<1, 256, 0, st>>>(fa);
    CU_OK(cudaGetLastError());
  }
  return 0;
}

extern "C" size_t zepp_meta_workspace_bytes(int R, int S, int K, int gpe) {
  const int tpt = kMetaThreads / K;
  const size_t tiles = (size_t)R * ((S + tpt - 1) / tpt);
  const size_t E = (size_t)R * gpe;
  return al(tiles * E * 4) + al(tiles * 2 * R * 4) + al((E + 1) * 4) + 4096;
}

extern "C" int zepp_dispatch_plan_words(int L, int NN) {
  const int nseg = L + NN - 1;
  return 8 + nseg + 1 + 3 * L + NN * (6 + 8 * L) + NN * (3 + L);
}

extern "C" int zepp_routed_meta(const int32_t* gathered, const int32_t* vce_in, int R, int L, int S, int K, int nlp,
                                int gpe, int my_rank, int direct, int relay_slots, const int64_t caps[8],
                                int copies_per_rank, int32_t* vce, float* probs_all, int32_t* splits,
                                int32_t* scatter_index, int32_t* sps, int32_t* uc, int64_t* demands, int64_t* dplan,
                                int64_t* cplan, void* ws, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (R < 1 || R > kMaxRanks || R % L) return fail("routed_meta: bad topology");
  if (K < 1 || K > 64) return fail("routed_meta: bad topk");
  const int E_virt = R * gpe, NN = R / L;
  if (E_virt > 4 * kMetaThreads) return fail("routed_meta: too many virtual experts");
  if (gathered && !probs_all) return fail("routed_meta: probs_all is required with gathered rows");
  MetaArgs m{};
  m.gathered = gathered; m.vce_in = vce_in; m.R = R; m.L = L; m.S = S; m.K = K; m.nlp = nlp; m.gpe = gpe;
  m.my_rank = my_rank;
  m.tokens_per_tile = kMetaThreads / K;
  m.tiles_per_src = (S + m.tokens_per_tile - 1) / m.tokens_per_tile;
  m.vce = vce; m.probs_all = probs_all; m.splits = splits; m.scatter_index = scatter_index; m.sps = sps; m.uc = uc;
  m.demands = (long long*)demands;
  for (int i = 0; i < 8; ++i) m.caps[i] = caps[i];
  m.direct = direct; m.relay_slots = relay_slots; m.dplan = (long long*)dplan; m.cplan = (long long*)cplan;
  m.copies_per_rank = copies_per_rank;
  uint8_t* w = (uint8_t*)ws;
  const size_t tiles = (size_t)R * m.tiles_per_src;
  m.tile_hist = (int*)w; w += al(tiles * E_virt * 4);
  m.tile_uc = (int*)w; w += al(tiles * 2 * R * 4);
  m.expert_base = (int*)w;
  m.n_tiles = nullptr; m.row_tok = nullptr; m.status = nullptr; m.routing_flags = nullptr; m.epoch_ptr = nullptr;
  uint8_t* wend = (uint8_t*)m.expert_base + al((size_t)(E_virt + 1) * 4);
  m.block_counter = (unsigned int*)wend;          // self-resetting arrival words at the end of the workspace
  m.grid_sync = (unsigned int*)wend + 2;
  const int grid = (int)tiles;
  const size_t sm = meta_smem(R, NN, E_virt);
  const size_t sm2 = pass2_smem(m.tokens_per_tile, K, E_virt);
  if (gpe > kMetaThreads) return fail("routed_meta: too many groups per rank");
  if (sm > 48 * 1024) return fail("routed_meta: too many ranks / experts");
  CU_OK(cudaMemsetAsync(m.block_counter, 0, 16, st));
  // one cooperative launch when every block of it can be resident at once, else two launches
  const size_t smf = meta_fused_smem_ints(R, NN, E_virt, m.tokens_per_tile, K) * sizeof(int);
  const char* off = getenv("ZEPP_B200_META_FUSED");
  if (smf <= 200 * 1024 && !(off != nullptr && off[0] == '0')) {
    int per_sm = 0, dev = 0, sms = 0;
    CU_OK(cudaGetDevice(&dev));
    CU_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (smf > 48 * 1024)
      CU_OK(cudaFuncSetAttribute(meta_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smf));
    CU_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, meta_fused_kernel, kMetaThreads, smf));
    if ((long long)per_sm * sms >= (long long)grid + 1) {
      FrontArgs f{};
      void* args[] = {(void*)&m, (void*)&f};
      CU_OK(cudaLaunchCooperativeKernel((const void*)meta_fused_kernel, dim3(grid + 1), dim3(kMetaThreads), args, smf, st));
      return 0;
    }
  }
  if (pass2_prepare(sm2)) return 1;
  meta_pass1_kernel<<<grid, kMetaThreads, sm, st>>>(m);
  CU_OK(cudaGetLastError());
  meta_pass2_kernel<<<grid, kMetaThreads, sm2, st>>>(m);
  CU_OK(cudaGetLastError());
  return 0;
}

static int swap_decide_prepare() {
  int dev = -1;
  CU_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  if (dev < 0 || dev >= kMaxDevices || !g_swap_attr[dev]) {
    CU_OK(cudaFuncSetAttribute(swap_decide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (dev >= 0 && dev < kMaxDevices) g_swap_attr[dev] = true;
  }
  return 0;
}

extern "C" int zepp_swap_decide_out_ints(int R, int G, int nlp, int cap) { return 3 + R + 4 * R * cap + R * nlp + G; }

static SwapArgs swap_args(const int* loads, int* p2l, int* l2p, const int* lcnts, int R, int G, int L, int nlp, double C,
                          int cap, int max_rounds, long long* out) {
  SwapArgs a{};
  a.loads = loads; a.p2l = p2l; a.l2p = l2p; a.lcnts = lcnts; a.R = R; a.G = G; a.L = L; a.nlp = nlp; a.cap = cap;
  a.max_rounds = max_rounds; a.C = C; a.out = out;
  return a;
}
static size_t swap_smem(int R, int G, int L, int nlp) {
  const int NS = R * nlp, NN = R / L, Q = NN * (L / 2) > 0 ? NN * (L / 2) : 1;
  return (size_t)(G + NS + R) * 8 + (size_t)(2 * NS + 7 * Q + NN + (kSwapThreads / 32) * 16 + 8) * 4;
}

extern "C" int zepp_swap_decide(const int32_t* loads, int32_t* p2l, int32_t* l2p, const int32_t* lcnts, int R, int G,
                                int L, int nlp, double C, int cap, int max_rounds, int64_t* out, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (R % L || L > kSwapMaxL) return fail("swap_decide: bad topology R=%d L=%d", R, L);
  const SwapArgs a = swap_args(loads, p2l, l2p, lcnts, R, G, L, nlp, C, cap, max_rounds, (long long*)out);
  const size_t sm = swap_smem(R, G, L, nlp);
  if (sm > 200 * 1024) return fail("swap_decide: tables too large for one block");
  if (swap_decide_prepare()) return 1;
  swap_decide_kernel<<<1, kSwapThreads, sm, st>>>(a);
  CU_OK(cudaGetLastError());
  return 0;
}

extern "C" int zepp_lane_arm(const int64_t* swap_out, int R, int rank, int nlp, int cap, int64_t* gate, int32_t* sched,
                             int64_t* ovr0, int64_t* ovr1, const int64_t* stag, int64_t epoch, void* stream) {
  lane_arm_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const long long*)swap_out, R, rank, nlp, cap, (long long*)gate,
                                                      sched, (long long*)ovr0, (long long*)ovr1,
                                                      (const long long*)stag, (long long)epoch, nullptr);
  CU_OK(cudaGetLastError());
  return 0;
}

__global__ void wait_geq_kernel(const unsigned long long* flag, unsigned long long value, unsigned long long limit_ns,
                                int* result) {
  if (threadIdx.x == 0) result[0] = wait_epoch_geq(flag, value, limit_ns) ? 1 : 0;
}

extern "C" int zepp_wait_geq(const uint64_t* flag, uint64_t value, int limit_ms, int32_t* result, void* stream) {
  if (limit_ms < 1 || limit_ms > 10000) return fail("wait_geq: limit must be 1..10000 ms");
  wait_geq_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const unsigned long long*)flag, value,
                                                      (unsigned long long)limit_ms * 1000000ull, result);
  CU_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------
// routed metadata without a caller-provided (or any) allocation
// ---------------------------------------------------------------------------------------------
// Some hosts of this library cannot allocate device memory at the point where they plan a step: a
// serving process that handed the whole GPU to its own memory pool at start-up (a cudaMalloc there
// fails, or stalls every stream behind its implicit device-wide synchronisation), or a planner
// thread that must never block on the allocator.  zepp_routed_meta needs a scratch workspace from
// its caller; this variant keeps the scratch in the library image instead: a fixed array in device
// global memory that every GPU loading the library holds until the process exits.
constexpr size_t kMetaScratchMaxBytes = 1u << 20;     // 1 MiB per GPU, the stated maximum
static __device__ __align__(256) unsigned char g_meta_scratch[kMetaScratchMaxBytes];

// In host code `g_meta_scratch` is only a handle of the symbol, never a device address: the
// address each GPU gave the array is asked for once per device (with that device current).
static void* g_meta_scratch_addr[kMaxRanks] = {};
static std::mutex g_meta_scratch_mutex;

extern "C" int zepp_routed_meta_noalloc(const int32_t* gathered, const int32_t* vce_in, int R, int L, int S, int K,
                                        int nlp, int gpe, int my_rank, int direct, int relay_slots,
                                        const int64_t caps[8], int copies_per_rank, int32_t* vce, float* probs_all,
                                        int32_t* splits, int32_t* scatter_index, int32_t* sps, int32_t* uc,
                                        int64_t* demands, int64_t* dplan, int64_t* cplan, void* stream) {
  if (R < 1 || R > kMaxRanks || L < 1 || R % L || S < 1 || K < 1 || K > 64 || gpe < 2)
    return fail("routed_meta_noalloc: bad shape R=%d L=%d S=%d K=%d gpe=%d", R, L, S, K, gpe);
  const size_t need = zepp_meta_workspace_bytes(R, S, K, gpe);
  if (need > kMetaScratchMaxBytes)
    return fail("routed_meta_noalloc: this routing needs %zu bytes of scratch, the built-in scratch holds %zu "
                "(R=%d S=%d K=%d gpe=%d); use zepp_routed_meta with a caller workspace",
                need, (size_t)kMetaScratchMaxBytes, R, S, K, gpe);
  int dev = -1;
  CU_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxRanks) return fail("routed_meta_noalloc: device ordinal %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_meta_scratch_mutex);
    if (g_meta_scratch_addr[dev] == nullptr) {
      // first call on this device: resolve the array's device address (not an allocation)
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_meta_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail("routed_meta_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      g_meta_scratch_addr[dev] = p;
    }
    scratch = g_meta_scratch_addr[dev];
  }
  // The scratch keeps the previous call's contents.  The only word that has to start at zero (the
  // block counter that elects the last metadata block) is cleared by zepp_routed_meta on the
  // stream at the start of every call; every other word a kernel of this call reads (tile
  // histograms, tile unique counts, expert bases) is written earlier in the same call.
  return zepp_routed_meta(gathered, vce_in, R, L, S, K, nlp, gpe, my_rank, direct, relay_slots, caps, copies_per_rank,
                          vce, probs_all, splits, scatter_index, sps, uc, demands, dplan, cplan, scratch, stream);
}
