// The grouped expert GEMMs on CTA pairs: two CTAs on neighbouring SMs (a cluster of two) drive one
// tcgen05.mma.cta_group::2 of M = 256 token rows x N = 256 weight rows per K step.  Each CTA stages ITS 128 token
// rows and ITS 128 weight rows (the gate block in the pair's first CTA and the up block in the second; or two
// neighbouring 128-feature blocks of W2) with ordinary, non-multicast TMA loads -- 32 KB per K step and CTA instead
// of the 48 KB a single CTA needs for the same 128 x 256 outputs, which is what bounds the single-CTA kernel
// (csrc/gemm.cuh) once an expert has hundreds of rows.  The tensor core reads the other CTA's half of the weight
// rows from that CTA's shared memory; every CTA accumulates its own 128 token rows x 256 features in its own TMEM,
// so the epilogues are those of the single-CTA kernel.
//
// Synchronisation inside a pair (all mbarriers; remote ones addressed through the cluster window):
//   full[stage]    on the LEADER (cluster rank 0): both producers arrive with their own byte counts and both CTAs'
//                  TMA loads complete on it; the leader's MMA thread waits for it;
//   empty[stage]   on BOTH CTAs: the leader's tcgen05.commit arrives on both once the MMAs have read the stage;
//   acc_full[a]    on BOTH CTAs (commit); acc_empty[a] on the leader, 8 arrivals (four epilogue warps per CTA).
// A cluster barrier separates barrier initialisation from the first remote arrival and the last use of the peer's
// shared memory from kernel exit; every path, aborted ones included, reaches both.
#pragma once
#include "common.cuh"
#include "gemm.cuh"

namespace zepp {

constexpr int kPairTileRows = 2 * kTileN;     // token rows of a pair's tile
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kWTileBytes + kXTileBytes;          // 32 KB: this CTA's weight rows + its token rows
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024;
constexpr int kPairAccCols = 2 * kTileN;                            // 256 fp32 columns per accumulator stage
constexpr int kPairTmemCols = kAccStages * kPairAccCols;            // 512

template <int MODE, bool LINES = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192 + 32 * kMaxGatherWarps, 1)
moe_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x32,
                     const __grid_constant__ CUtensorMap tm_x64, const __grid_constant__ CUtensorMap tm_x128,
                     const GemmArgs a) {
  static_assert(MODE == MODE_GATE_UP_SWIGLU || MODE == MODE_DOWN_COMBINE, "the pair kernel computes two weight blocks per item");
  static_assert(!LINES || MODE == MODE_DOWN_COMBINE, "line staging belongs to the combine epilogue");
  constexpr int STAGES = kPairStages;
  constexpr int kFeatPerItem = (MODE == MODE_DOWN_COMBINE) ? 2 * kTileM : kTileM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full_bar[kAccStages];
  __shared__ __align__(8) uint64_t acc_empty_bar[kAccStages];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ int s_row0[kMaxTilesSmem], s_gr[kMaxTilesSmem];      // first row; (group << 9) | rows (1..256)
  __shared__ int s_pref[kMaxTilesSmem + 1];                        // rows before tile i in schedule order
  __shared__ uint4 s_lines[LINES ? 4 : 1][LINES ? 256 : 1];        // per epilogue warp: 32 rows x 8 units of 16 bytes

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();                  // 0: the pair's leader
  const bool leader = cta == 0;
  const int pair = (int)blockIdx.x >> 1;
  const int n_pairs = (int)gridDim.x >> 1;
  const unsigned long long epoch = a.epoch_ptr != nullptr ? *a.epoch_ptr : 0ull;
  const bool violation = a.status != nullptr && a.status[ST_VIOLATION] != 0ull;
  int n_tiles = violation ? 0 : *a.tt.n_tiles;           // a step over capacity computes nothing
  if (n_tiles > kMaxTilesSmem) n_tiles = kMaxTilesSmem;
  const int total_items = n_tiles * a.n_feat_tiles;
  const int k_blocks = a.k_extent / kTileK;
  // balanced persistent schedule over the pairs
  const int rounds = (total_items + n_pairs - 1) / n_pairs;
  const int active_pairs = rounds > 0 ? (total_items + rounds - 1) / rounds : 1;
  const int item_stride = active_pairs;
  const int item_first = pair < active_pairs ? pair : total_items;
  for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
    s_row0[i] = a.tt.tile_row0[i];
    s_gr[i] = (a.tt.tile_group[i] << 9) | (a.tt.tile_rows[i] & 0x1FF);
  }
  if (MODE != MODE_DOWN_COMBINE && a.gather && warp == 2) {
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
      mbar_init(&full_bar[s], 2);            // one arrival (with its byte count) per CTA of the pair
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 8);       // four epilogue warps of each CTA
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_smem, kPairTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x32);
    tma_prefetch_desc(&tm_x64);
    tma_prefetch_desc(&tm_x128);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                        // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abortp = &abort_flag;
  const uint32_t peer_abort = map_to_cta(smem_u32(&abort_flag), cta ^ 1u);
  const uint32_t lead_full = map_to_cta(smem_u32(&full_bar[0]), 0u);            // + 8 * stage
  const uint32_t lead_acc_empty = map_to_cta(smem_u32(&acc_empty_bar[0]), 0u);  // + 8 * accumulator stage

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA of the pair)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int item = item_first; item < total_items && !*abortp; item += item_stride) {
        const int ti = item / a.n_feat_tiles;
        const int j = item - ti * a.n_feat_tiles;
        const int grp = s_gr[ti] >> 9;
        const int rows = s_gr[ti] & 0x1FF;
        const int row0 = s_row0[ti] + (int)cta * kTileN;               // this CTA's half of the tile
        const int my_rows = min(kTileN, max(0, rows - (int)cta * kTileN));
        const CUtensorMap* tmx = my_rows <= 32 ? &tm_x32 : (my_rows <= 64 ? &tm_x64 : &tm_x128);
        const uint32_t x_bytes = my_rows == 0 ? 0u : (my_rows <= 32 ? 32u : (my_rows <= 64 ? 64u : 128u)) * (kTileK * 2);
        const uint32_t tx = kWTileBytes + x_bytes;
        // this CTA's 128 weight rows: the first block of the item (gate / W2 block 2j) or the second (up / 2j+1)
        const int w_row = grp * a.w_rows_per_group + j * kFeatPerItem + (int)cta * a.up_row_offset;
        bool ok = true;
        if (a.swap_block != nullptr && grp >= a.n_groups) {
          // weights of an expert that arrives this step: wait for all of its chunks in the staging group
          const unsigned int need = (unsigned int)((a.w_vec + kSwapChunkVecs - 1) / kSwapChunkVecs);
          const unsigned int* cnt = a.w_ready + (grp - a.n_groups);
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu_u32(cnt) < need) {
            if (*abortp || globaltimer_ns() - t0 > a.flag_limit_ns) {
              record_timeout(a.status, WAIT_WEIGHTS, grp - a.n_groups, (long long)epoch);
              ok = false;
              break;
            }
            __nanosleep(128);
          }
        }
        if (ok && MODE != MODE_DOWN_COMBINE && a.gather && my_rows > 0) {
          // the tile's rows are assembled by gather warps (of any CTA): wait until all have landed
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu_u32(a.tile_ready + ti) < (unsigned int)rows) {
            if (*abortp || globaltimer_ns() - t0 > a.flag_limit_ns) {
              record_timeout(a.status, WAIT_TILE_READY, ti, (long long)epoch);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (item == item_first) trace_mark_max(a.status, TR_FIRST_ITEMS);
        }
        if (!ok) {
          abort_flag = 1;
          st_shared_cluster_u32(peer_abort, 1u);
          break;
        }
        fence_proxy_async();          // generic-proxy writes of gather / mover warps -> async-proxy TMA reads
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abortp, a.mbar_limit_ns)) {
            record_timeout(a.status, WAIT_MBAR_EMPTY, item, kb);
            abort_flag = 1;
            st_shared_cluster_u32(peer_abort, 1u);
            break;
          }
          uint8_t* st = smem + stage * kPairStageBytes;
          const uint32_t bar = lead_full + 8u * (uint32_t)stage;
          mbar_arrive_expect_tx_cluster(bar, tx);
          tma_load_2d_pair(st, &tm_w, bar, kb * kTileK, w_row);
          if (x_bytes != 0u) tma_load_2d_pair(st + kWTileBytes, tmx, bar, kb * kTileK, row0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (the pair's leader only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      const uint32_t idesc = make_idesc_bf16(2u * kTileN, 2u * kTileM);     // M = 256 token rows, N = 256 weight rows
      for (int item = item_first; item < total_items && !*abortp; item += item_stride) {
        if (!mbar_wait_bounded(&acc_empty_bar[acc], acc_phase ^ 1, abortp, a.mbar_limit_ns)) {
          record_timeout(a.status, WAIT_TMEM_EMPTY, item, acc);
          abort_flag = 1;
          st_shared_cluster_u32(peer_abort, 1u);
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * kPairAccCols;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abortp, a.mbar_limit_ns)) {
            record_timeout(a.status, WAIT_MBAR_FULL, item, kb);
            abort_flag = 1;
            st_shared_cluster_u32(peer_abort, 1u);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t wd = make_kmajor_sw128_desc(st);                    // 128 weight rows in each CTA
          const uint64_t xd = make_kmajor_sw128_desc(st + kWTileBytes);      // 128 token rows in each CTA
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) umma_bf16_pair(d0, xd + 2 * k, wd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);      // both CTAs' stages reusable once these MMAs have read them
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&acc_full_bar[acc]);       // both CTAs' accumulators complete
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (4 warps per CTA, own TMEM)
    const int quad = warp & 3;
    if (MODE != MODE_DOWN_COMBINE && a.gather) {
      // no accumulator can be ready before the step's rows are assembled: help assemble them first
      const int spare = (int)(blockDim.x >> 5) - 6;
      gemm_spare_warps<MODE>(a, s_pref, s_row0, n_tiles, warp, lane, epoch, &abort_flag, spare + (warp - 2), spare + 4, false);
    }
    const int tok = (int)cta * kTileN + quad * 32 + lane;           // token row inside the pair's tile
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int item = item_first; item < total_items; item += item_stride) {
      const int ti = item / a.n_feat_tiles;
      const int j = item - ti * a.n_feat_tiles;
      const int row0 = s_row0[ti];
      const int rows = s_gr[ti] & 0x1FF;
      const bool mine = tok < rows;
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
          if (out != nullptr) out += j * kFeatPerItem;
        }
      }
      int got = 1;
      if (lane == 0) {
        got = mbar_wait_bounded(&acc_full_bar[acc], acc_phase, abortp, a.mbar_limit_ns) ? 1 : 0;
        if (!got && !*abortp) {
          record_timeout(a.status, WAIT_TMEM_FULL, item, acc);
          abort_flag = 1;
          st_shared_cluster_u32(peer_abort, 1u);
        }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      if ((int)cta * kTileN + quad * 32 < rows) {      // warps whose 32 token rows are all padding skip the reads
        const uint32_t t0 = tmem_base + acc * kPairAccCols + ((uint32_t)(quad * 32) << 16);
        gemm_epilogue_rows<MODE, LINES>(a, t0, out, scale, j, lane, LINES ? s_lines[warp - 2] : nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_acc_empty + 8u * (uint32_t)acc);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    gemm_spare_warps<MODE>(a, s_pref, s_row0, n_tiles, warp, lane, epoch, &abort_flag, warp - 6,
                           (int)(blockDim.x >> 5) - 6 + (MODE != MODE_DOWN_COMBINE ? 4 : 0), true);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // the leader's MMAs no longer read this CTA's shared memory; no arrival is in flight
  if (threadIdx.x == 0) trace_mark_max(a.status, MODE == MODE_DOWN_COMBINE ? TR_GEMM2_END : TR_GEMM1_END);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
  if (MODE == MODE_DOWN_COMBINE && a.done_flags != nullptr) {
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
