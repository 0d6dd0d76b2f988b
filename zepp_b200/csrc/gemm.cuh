// Grouped expert GEMMs of the MoE layer on tcgen05 / TMEM (sm_100a).
//
// A tile of up to 128 routed token rows of one expert is the M side of the MMA (TMEM lanes), the
// expert's weight rows are the N side: one M128 x N256 x K16 instruction per K step covers the gate
// and the up block of W1 (dispatch GEMM) or two neighbouring 128-feature blocks of W2 (combine
// GEMM).  Both operands are K-major as stored.  D[token, feature] accumulates in TMEM in fp32, two
// accumulator stages of 256 columns, so the epilogue of one item runs under the MMAs of the next.
// With few rows per expert (decode: 32 rows at 512 tokens per rank) the kernel is bound by streaming
// each weight panel once from HBM and the unused MMA rows cost nothing; with many rows it is bound
// by shared-memory bandwidth (operand reads of the MMAs + TMA fills), which is why one N = 256
// instruction replaces two N = 128 ones that would each re-read the token tile.
//
//   dispatch GEMM  (replaces src/dispatch/cutlass_impls/ag_scatter_gemm_grouped_with_absmax.h:420-731
//                   + python/zepp/layer.py:20-27): the epilogue applies SwiGLU to the gate / up
//                   columns of a token and writes bf16 activations [row, I].
//   combine GEMM   (replaces src/combine/cutlass_impls/gather_rs_gemm_grouped_with_absmax.h and
//                   src/combine/combine_kernels.cu:106-304): the epilogue multiplies a token's row by
//                   the copy's top-k weight and stores the bf16 row slice straight into the home
//                   rank's [S, K, H] slot panel (a peer-mapped pointer over NVLink).
//
// One persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2..5 = epilogue (one TMEM lane quadrant = 32 token rows each; a thread owns one token and
// writes contiguous pieces of its row).  Optional warps 6.. (dispatch GEMM, fused mode) assemble the
// routed token rows in the local receive buffer, tile by tile in schedule order, and publish
// per-tile ready counters that the producer waits on before it issues the tile's TMA loads.
#pragma once
#include "common.cuh"

namespace zepp {

constexpr int kTileM = 128;       // output features per weight block (128 TMEM columns)
constexpr int kTileN = 128;       // token rows per tile (TMEM lanes)
constexpr int kTileK = 64;        // bf16 elements per smem row = 128 bytes = one swizzle row
constexpr int kWTileBytes = kTileM * kTileK * 2;   // 16 KB
constexpr int kXTileBytes = kTileN * kTileK * 2;   // 16 KB
constexpr int kAccStages = 2;
constexpr int kMaxGatherWarps = 8;     // warps 6.. of a dispatch GEMM CTA in fused mode (4 or 8, chosen at launch)
constexpr int kMaxTilesSmem = 1024;   // token tiles of one rank and step held in shared memory
constexpr int kSwapChunkVecs = 2048;  // 16-byte vectors a mover warp copies per credit (32 KB)

// -DZEPP_GEMM_PROFILE: CTA 0 of the dispatch GEMM sums, in SM cycles, how long its MMA thread waited for
// operand stages and for a free accumulator, and how long an epilogue warp worked and waited for
// accumulators (status words TR_PROF_*).  Off in the shipped library.
#ifdef ZEPP_GEMM_PROFILE
#define ZEPP_PROF(...) __VA_ARGS__
#else
#define ZEPP_PROF(...)
#endif

enum GemmMode : int { MODE_GATE_UP_SWIGLU = 0, MODE_SINGLE_GELU = 1, MODE_DOWN_COMBINE = 2 };

// Per-step tables written by the metadata kernels (device memory; nothing is read on the host).
struct TileTables {
  const int* n_tiles;      // [1] token tiles of this rank's experts this step
  const int* tile_group;   // [max_tiles] local group (1..gpe-1) of the tile
  const int* tile_row0;    // [max_tiles] first row of the tile in the receive / activation buffer
  const int* tile_rows;    // [max_tiles] valid rows (1..128)
};

struct GemmArgs {
  TileTables tt;
  int k_extent;            // H (dispatch GEMM) or I (combine GEMM)
  int n_feat_tiles;        // items per token tile: I/128 (dispatch GEMM) or ceil(H/256) (combine GEMM)
  int w_rows_per_group;    // rows of one expert's weight matrix: 2I, I or H
  int up_row_offset;       // weight rows between an item's two blocks: I (gate -> up) or 128 (next block of W2)
  // dispatch GEMM output
  __nv_bfloat16* act;      // [cap, ld_act]
  int ld_act;
  // combine GEMM epilogue
  const float* row_scale;          // [cap] top-k weight of the copy in row r
  const long long* row_dst;        // [cap] home * 2^40 + element offset into the home's panel
  __nv_bfloat16* const* panels;    // [W] peer-mapped slot panels [S*K, H]
  __nv_bfloat16* staging;          // unfused combine: rows go to staging[r, H] instead of the panels
  // completion signal of the combine GEMM (last CTA stores `epoch` into every peer's flag[rank])
  unsigned long long* const* done_flags;   // [W] peer-mapped flag arrays, or nullptr
  unsigned int* cta_counter;               // self-resetting arrival counter
  int world, rank;
  const unsigned long long* epoch_ptr;     // device step counter (the step's epoch; parity picks x buffers)
  // fused gather (dispatch GEMM, overlap strategy)
  const int* row_tok;                      // [cap] global token id (source * S + token) of row r
  const __nv_bfloat16* const* x_ptrs;      // [W] peer-mapped x buffers [S, H] of even epochs
  const __nv_bfloat16* const* x_ptrs_odd;  // ... of odd epochs
  const __nv_bfloat16* x_self;             // this rank's own x (read in place), or nullptr
  const unsigned long long* x_flags;       // [W] local flags: x of source s published for `epoch`
  __nv_bfloat16* recv;                     // [cap, H] local receive buffer (TMA source)
  unsigned int* tile_ready;                // [max_tiles] rows landed per tile (zeroed per step)
  int tokens_per_rank;
  int gather;                              // 1: run the gather warps and gate tiles on tile_ready
  // expert swap: this step's incoming experts (the decision's result block) are pulled from their source ranks'
  // slots into the staging groups that follow the slot groups of the weight tensor by this kernel's spare warps,
  // while the tiles of every other group compute; a tile of a staging group waits for its expert's chunks
  // (replaces the weight lanes of python/zepp/swap.py:464-559 and src/planner/lane_device.cu:82-163, and their
  // gate words polled by the GEMMs' tile loops)
  const long long* swap_block;             // nullptr: no swap in this layer
  int swap_ranks, swap_cap;                // R and moves per rank of the block's layout
  int n_groups;                            // gpe: groups >= n_groups are staging entries
  const uint4* const* w_peers;             // [W] peers' slot bases of this GEMM's weight matrix
  uint4* w_slots;                          // this rank's base of the same tensor (slots, then staging)
  unsigned long long w_vec;                // 16-byte vectors of one group
  unsigned int* w_ready;                   // [cap] chunks landed per staging entry (zeroed by the decision kernel)
  // bounded waits
  unsigned long long* status;
  unsigned long long mbar_limit_ns;   // inner (mbarrier) waits enclose the cross-rank waits: bounded later than those
  unsigned long long flag_limit_ns;
};

template <int MODE>
struct GemmCfg {
  // two weight tiles share one token tile per stage: gate | up rows of W1, or two neighbouring
  // 128-feature blocks of W2 (halves the token-tile bytes each flop pulls out of L2 / HBM)
  static constexpr bool kDual = (MODE == MODE_GATE_UP_SWIGLU || MODE == MODE_DOWN_COMBINE);
  static constexpr int kFeatPerItem = (MODE == MODE_DOWN_COMBINE) ? 2 * kTileM : kTileM;   // output features of an item
  static constexpr int kStageBytes = (kDual ? 2 : 1) * kWTileBytes + kXTileBytes;
  static constexpr int kStages = kDual ? 4 : 6;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;   // + alignment slack
  static constexpr int kAccCols = kDual ? 2 * kTileN : kTileN;      // TMEM columns per accumulator stage
  static constexpr int kTmemCols = kAccStages * kAccCols;           // 512 or 256
};

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// SwiGLU with the reference's rounding points (python/zepp/layer.py:20-27 on bf16 tensors;
// src/planner/lane_device.cu:476-501): both GEMM outputs are bf16, s = bf16(g / (1 + exp(-g))),
// out = bf16(float(s) * float(u)).
__device__ __forceinline__ __nv_bfloat16 swiglu_bf16(float gate_acc, float up_acc) {
  const float g = bf16_round(gate_acc);
  const float u = bf16_round(up_acc);
  const float s = bf16_round(__fdividef(g, 1.0f + __expf(-g)));   // 2-ulp fp32 quotient, then rounded to bf16
  return __float2bfloat16_rn(s * u);
}
__device__ __forceinline__ __nv_bfloat16 gelu_bf16(float acc) {
  const float h = bf16_round(acc);
  return __float2bfloat16_rn(0.5f * h * (1.0f + erff(h * 0.70710678118654752f)));
}

// Epilogue of one accumulator quadrant: thread <-> token row (TMEM lane), `t0` = TMEM address of the quadrant's
// first column of the item, `out` = where this token's 128 / 256 output features start (nullptr: padding row).
template <int MODE, bool LINES>
__device__ __forceinline__ void gemm_epilogue_rows(const GemmArgs& a, uint32_t t0, __nv_bfloat16* out, float scale, int j,
                                                   int lane, uint4* stg) {
  constexpr int kFeatPerItemE = (MODE == MODE_DOWN_COMBINE) ? 2 * kTileM : kTileM;
  if (MODE == MODE_GATE_UP_SWIGLU) {
    for (int c0 = 0; c0 < kTileM; c0 += 32) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(t0 + c0, g);
      tmem_ld_32x32(t0 + kTileM + c0, u);
      tmem_ld_wait();
      if (out != nullptr) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int n = q * 16 + e * 2;
            const __nv_bfloat162 p = __halves2bfloat162(
                swiglu_bf16(__uint_as_float(g[n]), __uint_as_float(u[n])),
                swiglu_bf16(__uint_as_float(g[n + 1]), __uint_as_float(u[n + 1])));
            w[e] = *reinterpret_cast<const uint32_t*>(&p);
          }
          st_global_v8(out + c0 + q * 16, w);
        }
      }
    }
  } else if (MODE == MODE_SINGLE_GELU) {
    for (int c0 = 0; c0 < kTileM; c0 += 32) {
      uint32_t g[32];
      tmem_ld_32x32(t0 + c0, g);
      tmem_ld_wait();
      if (out != nullptr) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int n = q * 16 + e * 2;
            const __nv_bfloat162 p = __halves2bfloat162(gelu_bf16(__uint_as_float(g[n])),
                                                        gelu_bf16(__uint_as_float(g[n + 1])));
            w[e] = *reinterpret_cast<const uint32_t*>(&p);
          }
          st_global_v8(out + c0 + q * 16, w);
        }
      }
    }
  } else {
    // reference rounding points (combine_kernels.cu:191-197): bf16 GEMM output, fp32 product with
    // the top-k weight, bf16 row on the wire.  64 features = 128 contiguous bytes per step.
    // An odd number of 128-feature blocks: the last item's second block lies past the expert's rows.
    const int feat_end = min(kFeatPerItemE, a.w_rows_per_group - j * kFeatPerItemE);
    for (int c0 = 0; c0 < feat_end; c0 += 64) {
      uint32_t g[32], h[32];
      tmem_ld_32x32(t0 + c0, g);
      tmem_ld_32x32(t0 + c0 + 32, h);
      tmem_ld_wait();
      if (LINES) {
        
#pragma unroll
        for (int q = 0; q < 8; ++q) {           // this row's 64 features as eight 16-byte units
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = (q & 3) * 8 + e * 2;
            const float v0 = __uint_as_float(q < 4 ? g[n] : h[n]);
            const float v1 = __uint_as_float(q < 4 ? g[n + 1] : h[n + 1]);
            const __nv_bfloat162 p = __floats2bfloat162_rn(bf16_round(v0) * scale, bf16_round(v1) * scale);
            w[e] = *reinterpret_cast<const uint32_t*>(&p);
          }
          stg[lane * 8 + (q ^ (lane & 7))] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {           // four rows per instruction, eight lanes per row
          const int r = 4 * i + (lane >> 3);
          const int q = lane & 7;
          const uint4 v = stg[r * 8 + (q ^ (r & 7))];
          __nv_bfloat16* po = reinterpret_cast<__nv_bfloat16*>(
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(out), r));
          if (po != nullptr) *reinterpret_cast<uint4*>(po + c0 + q * 8) = v;
        }
        __syncwarp();                           // the next 64 features reuse the staging
      } else if (out != nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int n = (q & 1) * 16 + e * 2;
            const float v0 = __uint_as_float(q < 2 ? g[n] : h[n]);
            const float v1 = __uint_as_float(q < 2 ? g[n + 1] : h[n + 1]);
            const __nv_bfloat162 p = __floats2bfloat162_rn(bf16_round(v0) * scale, bf16_round(v1) * scale);
            w[e] = *reinterpret_cast<const uint32_t*>(&p);
          }
          st_global_v8(out + c0 + q * 16, w);
        }
      }
    }
  }
}

// Warps 6.. of a GEMM CTA: the fused dispatch gather (dispatch GEMM, overlap strategy), then the pull of a swap's
// incoming experts.  `abort_flag` is the CTA-wide flag the other roles poll.
// `gw` of `gather_warps`: this warp's place among the CTA's gathering warps (the spare warps, and -- before their
// first accumulator can possibly be ready -- the four epilogue warps).
template <int MODE>
__device__ __forceinline__ void gemm_spare_warps(const GemmArgs& a, const int* s_pref, const int* s_row0, int n_tiles,
                                                 int warp, int lane, unsigned long long epoch, int* abort_flag_p,
                                                 int gw, int gather_warps, bool movers) {
  volatile int* abortp = abort_flag_p;
  // ------------------------------------------------------------------ gather warps (fused dispatch)
  if (MODE != MODE_DOWN_COMBINE && a.gather) {
    // every source must have published its x for this step
    bool ok = true;
    if (a.x_flags != nullptr && lane < a.world) {
      if (!wait_epoch_geq(a.x_flags + lane, epoch, a.flag_limit_ns)) {
        record_timeout(a.status, WAIT_X, lane, (long long)epoch);
        ok = false;
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (blockIdx.x == 0 && gw == 0 && lane == 0) trace_mark(a.status, TR_GEMM1_X);
    if (!ok) {
      if (lane == 0) *abort_flag_p = 1;
    } else {
      // Rows are pulled in schedule order: row q of the step belongs to gather warp (q mod all
      // gather warps), so every SM keeps loads in flight.  A warp first lists up to 32 of its rows
      // (lane j keeps the j-th), fetches their source tokens in one round trip, then streams the
      // rows two at a time.
      const int vec_per_row = a.k_extent / 8;                 // 16-byte vectors per row
      const int n_warps = gridDim.x * gather_warps;
      const int my_warp = blockIdx.x * gather_warps + gw;
      const int total_rows = s_pref[n_tiles];
      for (int g0 = my_warp; g0 < total_rows; g0 += 32 * n_warps) {
        {
          {
            // lane j takes this warp's j-th row of the list: a binary search of the prefix table
            const int g = g0 + lane * n_warps;
            int my_r = -1, my_ti = 0;
            if (g < total_rows) {
              int lo = 0, hi = n_tiles - 1;
              while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_pref[mid] <= g) lo = mid; else hi = mid - 1;
              }
              my_ti = lo;
              my_r = s_row0[lo] + (g - s_pref[lo]);
            }
            const int cnt = __popc(__ballot_sync(0xffffffffu, g < total_rows));
            const int n = cnt;
            const int tok = lane < n ? a.row_tok[my_r] : -1;
            // two rows at a time (16 x 512 bytes of loads in flight per warp); a fence and the tile
            // credits after every pair, so early tiles are complete early
            for (int j0 = 0; j0 < n; j0 += 2) {
              const int j1 = j0 + 2 < n ? j0 + 2 : n;
              for (int j = j0; j < j1; j += 2) {
                const uint4* srcA = nullptr;
                const uint4* srcB = nullptr;
                uint4* dstA = nullptr;
                uint4* dstB = nullptr;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int rr = __shfl_sync(0xffffffffu, my_r, (j + h) & 31);
                  const int tk = __shfl_sync(0xffffffffu, tok, (j + h) & 31);
                  if (j + h < j1) {
                    const int src = tk >= 0 ? tk / a.tokens_per_rank : -1;
                    if (src >= 0 && src < a.world) {
                      const int t = tk - src * a.tokens_per_rank;
                      const __nv_bfloat16* xb = (src == a.rank && a.x_self != nullptr)
                                                    ? a.x_self : ((epoch & 1) ? a.x_ptrs_odd[src] : a.x_ptrs[src]);
                      const uint4* sp = reinterpret_cast<const uint4*>(xb + (size_t)t * a.k_extent);
                      uint4* dp = reinterpret_cast<uint4*>(a.recv + (size_t)rr * a.k_extent);
                      if (h == 0) { srcA = sp; dstA = dp; } else { srcB = sp; dstB = dp; }
                    } else if (lane == 0 && a.status != nullptr) {
                      atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
                    }
                  }
                }
                for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
                  uint4 ba[8], bb[8];
#pragma unroll
                  for (int q = 0; q < 8; ++q) {
                    const int v = v0 + q * 32 + lane;
                    if (v < vec_per_row) {
                      if (srcA != nullptr) ba[q] = srcA[v];
                      if (srcB != nullptr) bb[q] = srcB[v];
                    }
                  }
#pragma unroll
                  for (int q = 0; q < 8; ++q) {
                    const int v = v0 + q * 32 + lane;
                    if (v < vec_per_row) {
                      if (dstA != nullptr) dstA[v] = ba[q];
                      if (dstB != nullptr) dstB[v] = bb[q];
                    }
                  }
                }
              }
              __threadfence();
              __syncwarp();
              if (lane >= j0 && lane < j1) atomicAdd(a.tile_ready + my_ti, 1u);
            }
          }
        }
      }
      if (lane == 0) trace_mark_max(a.status, TR_GATHER_END);
    }
  }
  if (movers && a.swap_block != nullptr && !*abortp) {
    // ---------------------------------------------------------------- movers (incoming experts of a swap)
    const long long rounds = a.swap_block[0];
    int cnt = rounds > 0 ? (int)a.swap_block[3 + a.rank] : 0;
    if (cnt > a.swap_cap) cnt = a.swap_cap;
    if (cnt > 0) {
      const long long* mv = a.swap_block + 3 + a.swap_ranks + (size_t)a.rank * a.swap_cap * 4;
      const int spare = (int)(blockDim.x >> 5) - 6;
      const unsigned long long n_warps = (unsigned long long)gridDim.x * spare;
      const unsigned long long me = (unsigned long long)blockIdx.x * spare + (warp - 6);
      const unsigned long long per = (a.w_vec + kSwapChunkVecs - 1) / kSwapChunkVecs;
      for (unsigned long long c = me; c < per * cnt; c += n_warps) {
        const int m = (int)(c / per);
        const unsigned long long v_lo = (c - (unsigned long long)m * per) * kSwapChunkVecs;
        const unsigned long long v_hi = v_lo + kSwapChunkVecs < a.w_vec ? v_lo + kSwapChunkVecs : a.w_vec;
        const int src_rank = (int)mv[4 * m + 1], src_slot = (int)mv[4 * m + 2];
        if (src_rank >= 0 && src_rank < a.world) {
          const uint4* sp = a.w_peers[src_rank] + (unsigned long long)(1 + src_slot) * a.w_vec;
          uint4* dp = a.w_slots + (unsigned long long)(a.n_groups + m) * a.w_vec;
          for (unsigned long long v0 = v_lo; v0 < v_hi; v0 += 256) {
            uint4 buf[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const unsigned long long v = v0 + q * 32 + lane;
              if (v < v_hi) buf[q] = sp[v];
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const unsigned long long v = v0 + q * 32 + lane;
              if (v < v_hi) dp[v] = buf[q];
            }
          }
        } else if (lane == 0 && a.status != nullptr) {
          atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(a.w_ready + m, 1u);
      }
    }
  }
}

// LINES (combine GEMM only): the epilogue writes whole 128-byte lines of the destination rows instead
// of 32-byte pieces.  Each epilogue warp stages its 32 token rows x 64 features in its own 4 KB of
// shared memory (16-byte units XOR-swizzled by the row, so neither the row-wise writes nor the
// line-wise reads conflict) and eight lanes then store one row's 128 contiguous bytes.  Meant for
// destination panels on peer GPUs, where NVLink carries a few large writes far better than many
// 32-byte ones.
template <int MODE, bool LINES = false>
__global__ void __launch_bounds__(192 + 32 * kMaxGatherWarps, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x32,
                const __grid_constant__ CUtensorMap tm_x64, const __grid_constant__ CUtensorMap tm_x128,
                const GemmArgs a) {
  using Cfg = GemmCfg<MODE>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full_bar[kAccStages];
  __shared__ __align__(8) uint64_t acc_empty_bar[kAccStages];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ int s_row0[kMaxTilesSmem], s_gr[kMaxTilesSmem];      // first row; (group << 9) | rows
  __shared__ int s_pref[kMaxTilesSmem + 1];                        // rows before tile i in schedule order
  static_assert(!LINES || MODE == MODE_DOWN_COMBINE, "line staging belongs to the combine epilogue");
  __shared__ uint4 s_lines[LINES ? 4 : 1][LINES ? 256 : 1];        // per epilogue warp: 32 rows x 8 units of 16 bytes

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const unsigned long long epoch = a.epoch_ptr != nullptr ? *a.epoch_ptr : 0ull;
  const bool violation = a.status != nullptr && a.status[ST_VIOLATION] != 0ull;
  int n_tiles = violation ? 0 : *a.tt.n_tiles;           // a step over capacity computes nothing
  if (n_tiles > kMaxTilesSmem) n_tiles = kMaxTilesSmem;   // (the host sizes max_tiles below this)
  const int total_items = n_tiles * a.n_feat_tiles;
  const int k_blocks = a.k_extent / kTileK;
  // balanced persistent schedule: the items are spread over the fewest CTAs that still finish in
  // ceil(items / grid) rounds, so no round runs with a mostly idle machine
  const int rounds = (total_items + (int)gridDim.x - 1) / (int)gridDim.x;
  const int active_ctas = rounds > 0 ? (total_items + rounds - 1) / rounds : 1;
  const int item_stride = active_ctas;
  const int item_first = (int)blockIdx.x < active_ctas ? (int)blockIdx.x : total_items;
  for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
    s_row0[i] = a.tt.tile_row0[i];
    s_gr[i] = (a.tt.tile_group[i] << 9) | (a.tt.tile_rows[i] & 0x1FF);
  }

  if (MODE != MODE_DOWN_COMBINE && a.gather && warp == 2) {
    // exclusive prefix of the tiles' row counts (read straight from the global table: the shared
    // copy above is filled by other threads and only ordered by the barrier below)
    int carry = 0;
    for (int i0 = 0; i0 < n_tiles; i0 += 32) {
      const int v = i0 + lane < n_tiles ? a.tt.tile_rows[i0 + lane] : 0;
      int incl = v;
      for (int off = 1; off < 32; off <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += u;
      }
      if (i0 + lane < n_tiles) s_pref[i0 + lane] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_pref[n_tiles] = carry;
  }
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) trace_mark(a.status, MODE == MODE_DOWN_COMBINE ? TR_GEMM2 : TR_GEMM1);
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 4);       // one arrival per epilogue warp
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x32);
    tma_prefetch_desc(&tm_x64);
    tma_prefetch_desc(&tm_x128);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int item = item_first; item < total_items && !*abortp; item += item_stride) {
        const int ti = item / a.n_feat_tiles;
        const int j = item - ti * a.n_feat_tiles;
        const int grp = s_gr[ti] >> 9;
        const int row0 = s_row0[ti];
        const int rows = s_gr[ti] & 0x1FF;
        const CUtensorMap* tmx = rows <= 32 ? &tm_x32 : (rows <= 64 ? &tm_x64 : &tm_x128);
        const uint32_t x_bytes = (rows <= 32 ? 32u : (rows <= 64 ? 64u : 128u)) * (kTileK * 2);
        const uint32_t tx = (Cfg::kDual ? 2u : 1u) * kWTileBytes + x_bytes;
        const int w_row = grp * a.w_rows_per_group + j * Cfg::kFeatPerItem;
        if (a.swap_block != nullptr && grp >= a.n_groups) {
          // weights of an expert that arrives this step: wait for all of its chunks in the staging group
          const unsigned int need = (unsigned int)((a.w_vec + kSwapChunkVecs - 1) / kSwapChunkVecs);
          const unsigned int* cnt = a.w_ready + (grp - a.n_groups);
          const unsigned long long t0 = globaltimer_ns();
          bool ok = true;
          while (ld_acquire_gpu_u32(cnt) < need) {
            if (*abortp || globaltimer_ns() - t0 > a.flag_limit_ns) {
              record_timeout(a.status, WAIT_WEIGHTS, grp - a.n_groups, (long long)epoch);
              ok = false;
              break;
            }
            __nanosleep(128);
          }
          if (!ok) {
            abort_flag = 1;
            break;
          }
          fence_proxy_async();        // the movers' generic-proxy stores -> TMA reads
        }
        int kb_first = 0;
        if (MODE != MODE_DOWN_COMBINE && a.gather) {
          // rows of this tile are pulled by gather warps (of any CTA).  If they have not all landed yet,
          // start streaming the weight tiles of the first stages, then wait, then add the token tiles
          if (ld_acquire_gpu_u32(a.tile_ready + ti) < (unsigned int)rows) {
            const int pre = k_blocks < STAGES ? k_blocks : STAGES;
            const int stage0 = stage;
            bool ok = true;
            for (int kb = 0; kb < pre && ok; ++kb) {
              if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abortp, a.mbar_limit_ns)) {
                record_timeout(a.status, WAIT_MBAR_EMPTY, item, kb);
                ok = false;
                break;
              }
              uint8_t* st = smem + stage * Cfg::kStageBytes;
              mbar_expect_tx(&full_bar[stage], tx);
              tma_load_2d(st, &tm_w, &full_bar[stage], kb * kTileK, w_row);
              if (Cfg::kDual) tma_load_2d(st + kWTileBytes, &tm_w, &full_bar[stage], kb * kTileK, w_row + a.up_row_offset);
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            const unsigned long long t0 = globaltimer_ns();
            while (ok && ld_acquire_gpu_u32(a.tile_ready + ti) < (unsigned int)rows) {
              if (*abortp || globaltimer_ns() - t0 > a.flag_limit_ns) {
                record_timeout(a.status, WAIT_TILE_READY, ti, (long long)epoch);
                ok = false;
                break;
              }
              __nanosleep(64);
            }
            if (!ok) {
              abort_flag = 1;
              break;
            }
            fence_proxy_async();      // generic-proxy writes of the gather -> async-proxy TMA reads
            int sx = stage0;
            for (int kb = 0; kb < pre; ++kb) {
              tma_load_2d(smem + sx * Cfg::kStageBytes + (Cfg::kDual ? 2 : 1) * kWTileBytes, tmx, &full_bar[sx],
                          kb * kTileK, row0);
              if (++sx == STAGES) sx = 0;
            }
            kb_first = pre;
          } else {
            fence_proxy_async();
          }
          if (item == item_first) trace_mark_max(a.status, TR_FIRST_ITEMS);
        }
        for (int kb = kb_first; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abortp, a.mbar_limit_ns)) {
            record_timeout(a.status, WAIT_MBAR_EMPTY, item, kb);
            abort_flag = 1;
            break;
          }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full_bar[stage], tx);
          tma_load_2d(st, &tm_w, &full_bar[stage], kb * kTileK, w_row);
          if (Cfg::kDual) tma_load_2d(st + kWTileBytes, &tm_w, &full_bar[stage], kb * kTileK, w_row + a.up_row_offset);
          tma_load_2d(st + (Cfg::kDual ? 2 : 1) * kWTileBytes, tmx, &full_bar[stage], kb * kTileK, row0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // tokens x (two weight blocks): one instruction per K step, whatever the tile's valid rows (rows
      // of the token tile beyond them hold stale shared memory and only reach accumulator rows that
      // the epilogue never reads)
      const uint32_t idesc = make_idesc_bf16_m128(Cfg::kDual ? 2u * kTileM : (uint32_t)kTileM);
      ZEPP_PROF(long long prof_data = 0; long long prof_acc = 0; long long prof_t;)
      for (int item = item_first; item < total_items && !*abortp; item += item_stride) {
        ZEPP_PROF(prof_t = clock64();)
        if (!mbar_wait_bounded(&acc_empty_bar[acc], acc_phase ^ 1, abortp, a.mbar_limit_ns)) {
          record_timeout(a.status, WAIT_TMEM_EMPTY, item, acc);
          abort_flag = 1;
          break;
        }
        ZEPP_PROF(prof_acc += clock64() - prof_t;)
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * Cfg::kAccCols;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ZEPP_PROF(prof_t = clock64();)
          if (!mbar_wait_bounded(&full_bar[stage], phase, abortp, a.mbar_limit_ns)) {
            record_timeout(a.status, WAIT_MBAR_FULL, item, kb);
            abort_flag = 1;
            ok = false;
            break;
          }
          ZEPP_PROF(prof_data += clock64() - prof_t;)
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t wd = make_kmajor_sw128_desc(st);     // 128 or 256 weight rows (the blocks are adjacent)
          const uint64_t xd = make_kmajor_sw128_desc(st + (Cfg::kDual ? 2 : 1) * kWTileBytes);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) umma_bf16(d0, xd + 2 * k, wd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);       // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full_bar[acc]);        // accumulator complete
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
      ZEPP_PROF(if (blockIdx.x == 0 && a.status != nullptr && MODE != MODE_DOWN_COMBINE) {
        a.status[TR_PROF_MMA_DATA] = (unsigned long long)prof_data; a.status[TR_PROF_MMA_ACC] = (unsigned long long)prof_acc; })
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (4 warps)
    // TMEM holds D[token, feature]: a thread owns one token row of the tile (the lane of its warp's
    // quadrant), reads 32 feature columns at a time and writes them as contiguous 16-byte vectors of
    // that token's output row.  Nothing is staged in shared memory and the warps never synchronise
    // with each other.
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
    if (MODE != MODE_DOWN_COMBINE && a.gather) {
      // no accumulator can be ready before the step's rows are assembled: help assemble them first
      const int spare = (int)(blockDim.x >> 5) - 6;
      gemm_spare_warps<MODE>(a, s_pref, s_row0, n_tiles, warp, lane, epoch, &abort_flag, spare + (warp - 2), spare + 4, false);
    }
    const int tok = quad * 32 + lane;           // token row inside the tile
    int acc = 0;
    uint32_t acc_phase = 0;
    ZEPP_PROF(long long prof_busy = 0; long long prof_wait = 0; long long prof_t = clock64();)
    for (int item = item_first; item < total_items; item += item_stride) {
      const int ti = item / a.n_feat_tiles;
      const int j = item - ti * a.n_feat_tiles;
      const int row0 = s_row0[ti];
      const int rows = s_gr[ti] & 0x1FF;
      const bool mine = tok < rows;
      // where this token's row goes (and its top-k weight): looked up while the item's MMAs still run
      __nv_bfloat16* out = nullptr;
      float scale = 0.f;
      if (mine) {
        if (MODE != MODE_DOWN_COMBINE) {
          out = a.act + (size_t)(row0 + tok) * a.ld_act + j * kTileM;
        } else {
          scale = a.row_scale[row0 + tok];
          if (a.staging != nullptr) {
            out = a.staging + (size_t)(row0 + tok) * a.w_rows_per_group;
          } else {
            const long long dst = a.row_dst[row0 + tok];
            if (dst >= 0) out = a.panels[(int)(dst >> 40)] + (size_t)(dst & ((1ll << 40) - 1));
          }
          if (out != nullptr) out += j * Cfg::kFeatPerItem;
        }
      }
      int got = 1;
      if (lane == 0) {
        got = mbar_wait_bounded(&acc_full_bar[acc], acc_phase, abortp, a.mbar_limit_ns) ? 1 : 0;
        if (!got && !*abortp) {
          record_timeout(a.status, WAIT_TMEM_FULL, item, acc);
          abort_flag = 1;
        }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      ZEPP_PROF(prof_wait += clock64() - prof_t; prof_t = clock64();)
      tc_fence_after();
      if (quad * 32 < rows) {                   // warps whose 32 token rows are all padding skip the reads
        const uint32_t t0 = tmem_base + acc * Cfg::kAccCols + ((uint32_t)(quad * 32) << 16);
        gemm_epilogue_rows<MODE, LINES>(a, t0, out, scale, j, lane, LINES ? s_lines[warp - 2] : nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      ZEPP_PROF(prof_busy += clock64() - prof_t; prof_t = clock64();)
    }
    ZEPP_PROF(if (blockIdx.x == 0 && warp == 2 && lane == 0 && a.status != nullptr && MODE != MODE_DOWN_COMBINE) {
      a.status[TR_PROF_EPI_BUSY] = (unsigned long long)prof_busy; a.status[TR_PROF_EPI_WAIT] = (unsigned long long)prof_wait; })
  } else {
    gemm_spare_warps<MODE>(a, s_pref, s_row0, n_tiles, warp, lane, epoch, &abort_flag, warp - 6,
                           (int)(blockDim.x >> 5) - 6 + (MODE != MODE_DOWN_COMBINE ? 4 : 0), true);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_mark_max(a.status, MODE == MODE_DOWN_COMBINE ? TR_GEMM2_END : TR_GEMM1_END);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (MODE == MODE_DOWN_COMBINE && a.done_flags != nullptr) {
    // the block barrier above ordered every thread's panel stores before thread 0; its fence makes
    // them visible system-wide before the CTA's arrival; the last CTA publishes the epoch
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicInc(a.cta_counter, gridDim.x - 1);
      if (prev == gridDim.x - 1) {
        __threadfence_system();
        for (int p = 0; p < a.world; ++p) st_relaxed_sys(a.done_flags[p] + a.rank, epoch);
      }
    }
  }
}

}  // namespace zepp
