// Routed metadata of a step: virtual group ids, per-expert counts, the deterministic stable
// scatter index, per-source splits, unique (token, destination) counts, exact buffer demands with
// their violation mask, the dispatch / combine plan heads, and the row / tile tables the two GEMM
// kernels read.  Replaces DispatchGemmOp::derive_routed_meta (src/dispatch/ths_op/dispatch_gemm.cc:916-1101;
// kernels src/dispatch/sort_util.cu:354-541, 957-1122, 1153-1500), planner_tail_kernel
// (src/planner/lane_device.cu:526-540) and the combine tables (src/combine/combine_kernels.cu:1308,1546);
// host references python/zepp/routing.py:306-331, python/zepp/capacity.py:30-55.
//
// No atomics on global memory beyond one arrival counter, no host read.  Three stages:
//   count  one block per tile of one source's entries: vce / probs_all (from the gathered routing
//          rows), per-tile expert histogram, per-tile unique owner / node counts;
//   scan   splits, sps, uc, exclusive bases, demands + mask, plan heads, this rank's tile schedule;
//   rank   stable rank of every copy inside its expert (warps of a tile take turns, lanes rank
//          themselves with match_any), scatter_index, and for copies owned by this rank the GEMM row
//          tables (source token, home slot, top-k weight).
// meta_fused_kernel runs all three in ONE cooperative launch (count -> grid barrier -> every tile block
// derives its own bases from the per-tile counts and ranks its copies, while one extra block writes the
// step's tables); meta_pass1_kernel (count + scan in its last block) and meta_pass2_kernel (rank) are the
// two-launch form for grids too large to be co-resident.
//
// A copy whose expert id is negative is a PAD copy (the rows a caller adds to fill a token bucket): it has
// no owner, is counted nowhere, moves no row and gets vce = scatter_index = -1.
#pragma once
#include "common.cuh"
#include "planner.cuh"

namespace zepp {

constexpr int kMetaThreads = 1024;
constexpr int kTileRowsMax = 128;

struct MetaArgs {
  // input: either the gathered routing rows [R, 2*SK] (phys | weight bits) or vce directly
  const int* gathered;
  const int* gathered_odd;  // odd-epoch copy when `epoch_ptr` is set
  const int* vce_in;
  // one rank with a single-replica placement: the routing is a slot lookup and is done here, the step's
  // first kernel (no routing launch, no exchange); local_topk = nullptr otherwise
  const int* local_topk;    // [SK] expert ids of this rank's tokens
  const float* local_probs; // [SK]
  const int* slot_of;       // [G] the only physical slot of every expert (-1: none)
  int G;
  int* phys_own;            // [SK] out
  int* send_row;            // [2*SK] out: phys | weight bits
  int* gathered_out;        // [2*SK] out: the same row in the gather table of this epoch's parity
  int* gathered_out_odd;
  unsigned long long* ctr;  // step counter committed by the last block
  int R, L, S, K, nlp, gpe, my_rank;
  int tokens_per_tile, tiles_per_src;
  // outputs
  int* vce;                 // [R*S*K]
  float* probs_all;         // [R*S*K] (only with `gathered`)
  int* splits;              // [E_virt]
  int* scatter_index;       // [R*S*K]
  int* sps;                 // [R, E_virt]
  int* uc;                  // [R, R+NN]
  long long* demands;       // [8]: 7 demands + violation mask
  long long caps[8];
  int direct, relay_slots;
  long long* dplan;         // dispatch plan head words of my_rank (or nullptr)
  long long* cplan;         // send_off[W+1] | send_rows[W] | dst_off[W] | lane_off[W+1] (or nullptr)
  int copies_per_rank;
  // workspace
  int* tile_hist;           // [R*tiles_per_src, E_virt]  -> tile bases after scan
  int* tile_uc;             // [R*tiles_per_src, R+NN]
  int* expert_base;         // [E_virt + 1]
  // GEMM tables of my_rank
  int* n_tiles;
  int* tile_group;
  int* tile_row0;
  int* tile_rows;
  unsigned int* tile_ready;
  int max_tiles;
  int recv_cap;
  int* m_this;              // [2]: rows this rank computes, first global row (m_start)
  int* row_tok;             // [recv_cap]
  long long* row_dst;       // [recv_cap]
  float* row_scale;         // [recv_cap]
  int hidden;               // H (row_dst is an element offset into the home's [S*K, H] panel)
  int staged;               // 1: row_tok holds (source, staging slot) instead of (source, token)
  const int* group_order;   // [gpe] schedule word per group (bit 30 = moved-in slot: its tiles go last) or nullptr
  int tile_rows_max;        // token rows of a GEMM tile: 128 (one CTA per tile) or 256 (CTA pairs); 0 = 128
  const int* group_redirect;// [gpe] group whose weights a group's tiles read (a staging entry for a moved-in slot) or nullptr
  // exchange wait
  const unsigned long long* routing_flags;
  const unsigned long long* epoch_ptr;
  unsigned long long limit_ns;
  unsigned long long* status;
  unsigned int* block_counter;   // pass1: the last block to finish runs the scan
  unsigned int* grid_sync;       // fused kernel: [0] self-resetting arrival counter, [1] release generation
};

__device__ void meta_scan_body(MetaArgs& a, int* chunks, bool bases_in_place);
__device__ void plan_heads(MetaArgs& a, const int* chunks, const int* s_uc);

// Virtual group of entry n of source `src` (-1: a pad copy).  Writes vce (and probs_all when the routing
// rows carry weights); on one rank with a single-replica placement it also does the slot lookup and
// writes the routing rows themselves.
__device__ __forceinline__ int meta_decode_entry(const MetaArgs& a, bool local, int src, int n, int SK, int E_virt) {
  const size_t flat = (size_t)src * SK + n;
  int v;
  if (local) {
    const int e = a.local_topk[n];
    int phys = -1;
    if (e >= a.G) {
      if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
    } else if (e >= 0 && (phys = a.slot_of[e]) < 0) {
      if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_ROUTE);
      phys = -1;
    }
    const float w = a.local_probs[n];
    a.phys_own[n] = phys;
    a.send_row[n] = phys; a.send_row[SK + n] = __float_as_int(w);
    a.gathered_out[n] = phys; a.gathered_out[SK + n] = __float_as_int(w);
    a.probs_all[flat] = w;
    v = phys < 0 ? -1 : (phys / a.nlp) * a.gpe + 1 + phys % a.nlp;
  } else if (a.gathered) {
    const int phys = a.gathered[(size_t)src * 2 * SK + n];
    v = phys < 0 ? -1 : (phys / a.nlp) * a.gpe + 1 + phys % a.nlp;
    a.probs_all[flat] = __int_as_float(a.gathered[(size_t)src * 2 * SK + SK + n]);
  } else {
    v = a.vce_in[flat];
    if (v < 0) v = -1;
  }
  if (v >= E_virt) {
    if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
    v = 0;
  }
  a.vce[flat] = v;
  return v;
}

__global__ void __launch_bounds__(kMetaThreads) meta_pass1_kernel(MetaArgs a) {
  extern __shared__ int sm[];
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, SK = a.S * a.K;
  int* hist = sm;                       // [E_virt]
  int* ucs = sm + E_virt;               // [R + NN]
  const bool local = a.local_topk != nullptr;
  const unsigned long long epoch = step_epoch(a.epoch_ptr, local);
  if (a.epoch_ptr != nullptr && (epoch & 1)) { a.gathered = a.gathered_odd; a.gathered_out = a.gathered_out_odd; }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (local) {
      trace_mark(a.status, TR_ROUTE);
      trace_mark(a.status, TR_RING + (int)(epoch & 15));
    }
    trace_mark(a.status, TR_PASS1);
  }
  if (!block_wait_all(a.routing_flags, R, epoch, a.limit_ns, a.status, WAIT_ROUTING)) return;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a.status, TR_PASS1_GO);
  const int src = blockIdx.x / a.tiles_per_src;
  const int tb = blockIdx.x - src * a.tiles_per_src;
  for (int i = threadIdx.x; i < E_virt + R + NN; i += blockDim.x) sm[i] = 0;
  __syncthreads();
  const int T = a.tokens_per_tile * a.K;
  const int n_lo = tb * T;
  const int n_hi = min(SK, n_lo + T);
  for (int n = n_lo + threadIdx.x; n < n_hi; n += blockDim.x) {
    const int v = meta_decode_entry(a, local, src, n, SK, E_virt);
    if (v >= 0) atomicAdd(&hist[v], 1);
  }
  __syncthreads();
  // unique owners / nodes per token (a token may pick one rank several times)
  const int t_lo = tb * a.tokens_per_tile;
  const int t_hi = min(a.S, t_lo + a.tokens_per_tile);
  for (int t = t_lo + threadIdx.x; t < t_hi; t += blockDim.x) {
    unsigned long long owners = 0, nodes = 0;
    for (int k = 0; k < a.K; ++k) {
      const int v = a.vce[((size_t)src * a.S + t) * a.K + k];
      if (v < 0) continue;                       // pad copy
      const int o = v / a.gpe;
      owners |= 1ull << o;
      nodes |= 1ull << (o / a.L);
    }
    while (owners) { const int o = __ffsll((long long)owners) - 1; owners &= owners - 1; atomicAdd(&ucs[o], 1); }
    while (nodes) { const int o = __ffsll((long long)nodes) - 1; nodes &= nodes - 1; atomicAdd(&ucs[R + o], 1); }
  }
  __syncthreads();
  int* th = a.tile_hist + (size_t)blockIdx.x * E_virt;
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) th[e] = hist[e];
  int* tu = a.tile_uc + (size_t)blockIdx.x * (R + NN);
  for (int i = threadIdx.x; i < R + NN; i += blockDim.x) tu[i] = ucs[i];
  // the last block to finish turns the per-tile counts into the step's tables (no extra launch)
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicInc(a.block_counter, gridDim.x - 1) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  meta_scan_body(a, sm, true);
  // every block has read the counter by now (they all arrived before this block was chosen)
  if (local && threadIdx.x == 0 && a.ctr != nullptr) *a.ctr = epoch;
}

// Exact demands of a step (python/zepp/capacity.py:30-55) from chunks[s][d] (rows from source s to
// destination d, shared memory) and the unique counts; run by one thread (R <= 64; the single-node
// case touches only the R x R chunk table).
__device__ void demands_from_chunks(const int* chunks, const int* uc, int W, int L, int relay_slots, int direct,
                                    const long long* caps, long long* out) {
  const int NN = W / L;
  long long recv_rows = 0, pair = 0;
  for (int d = 0; d < W; ++d) {
    long long col = 0;
    for (int s = 0; s < W; ++s) {
      const long long ch = chunks[s * W + d];
      col += ch;
      if (ch > pair) pair = ch;
    }
    if (col > recv_rows) recv_rows = col;
  }
  long long dem[7] = {recv_rows, recv_rows, 1, 1, 1, 1, pair};
  if (NN > 1) {
    const int ucw = W + NN;
    long long disp = recv_rows;
    for (int d = 0; d < W; ++d) {
      long long tot = 0;
      for (int s = 0; s < W; ++s) tot += (s / L == d / L) ? uc[s * ucw + d] : uc[s * ucw + W + d / L];
      if (tot > disp) disp = tot;
    }
    long long stage = 0, relay = 0, conv = 0, wire = 0;
    for (int n = 0; n < NN; ++n) {
      for (int k = 0; k < L; ++k) {
        long long st = 0, cv = 0, wr = 0;
        for (int ns = 0; ns < NN; ++ns) {
          if (ns == n) continue;
          long long T = 0;
          for (int l = 0; l < L; ++l) T += uc[(ns * L + l) * ucw + W + n];
          const long long chunk = T / L + (k < T % L ? 1 : 0);
          st += chunk;
          if (chunk > relay) relay = chunk;
          for (int ls = 0; ls < L; ++ls) cv += chunks[(ns * L + k) * W + n * L + ls];
          wr += uc[(ns * L + k) * ucw + W + n];
        }
        if (st > stage) stage = st;
        if (cv > conv) conv = cv;
        if (wr > wire) wire = wr;
      }
    }
    dem[1] = disp; dem[2] = stage; dem[3] = relay * relay_slots; dem[4] = conv; dem[5] = wire;
  }
  long long mask = 0;
  for (int i = 0; i < 7; ++i) { if (dem[i] < 1) dem[i] = 1; out[i] = dem[i]; }
  if (direct) {
    if (dem[0] > caps[0]) mask |= 1;
    if (dem[6] > caps[7]) mask |= 0x80;
  } else {
    const int di[7] = {0, 1, 2, 3, 0, 4, 5};
    for (int b = 0; b < 7; ++b)
      if (dem[di[b]] > caps[b]) mask |= 1ll << b;
  }
  out[7] = mask;
}

__device__ __forceinline__ long long region_rows(const int* uc, int W, int L, int s, int d) {
  const int NN = W / L;
  return (s / L == d / L) ? uc[s * (W + NN) + d] : uc[s * (W + NN) + W + d / L];
}

// block-wide exclusive scan of one int per thread (blockDim.x <= 1024); returns the exclusive
// prefix, *total gets the sum
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot, int* total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int incl = v;
  #pragma unroll 1
  for (int off = 1; off < 32; off <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += u;
  }
  __syncthreads();
  if (lane == 31) warp_tot[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    const int t = lane < (int)(blockDim.x >> 5) ? warp_tot[lane] : 0;
    int inc2 = t;
    #pragma unroll 1
    for (int off = 1; off < 32; off <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc2, off);
      if (lane >= off) inc2 += u;
    }
    warp_tot[lane] = inc2 - t;
    if (lane == 31) warp_tot[32] = inc2;
  }
  __syncthreads();
  *total = warp_tot[32];
  return warp_tot[wid] + incl - v;
}

// Shared memory of the scan (ints): chunks[R*R] (rows from source s to destination rank d) |
// uc[R*(R+NN)] | splits[E_virt] | base[E_virt+1].  Everything later stages read comes from these
// copies, so the block goes to global memory once to read the per-tile counts and once to write.
__host__ __device__ inline size_t meta_scan_smem_ints(int R, int NN, int E_virt) {
  return (size_t)R * R + (size_t)R * (R + NN) + 2 * (size_t)E_virt + 1;
}

__device__ void meta_scan_body(MetaArgs& a, int* sm, bool bases_in_place) {
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, ucw = R + NN;
  const int n_blocks = R * a.tiles_per_src;
  int* chunks = sm;
  int* s_uc = chunks + R * R;
  int* s_splits = s_uc + R * ucw;
  int* s_base = s_splits + E_virt;
  __shared__ int warp_tot[33];
  __shared__ long long viol;
  __syncthreads();
  if (threadIdx.x == 0) trace_mark(a.status, TR_SCAN);
  #pragma unroll 1
  for (int i = threadIdx.x; i < R * R; i += blockDim.x) chunks[i] = 0;
  #pragma unroll 1
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) s_splits[e] = 0;
  __syncthreads();
  // per source splits, totals, chunk table: one (source, expert) pair per thread, its tiles' counts loaded
  // independently of each other (the loop is unrolled so that the loads are in flight together)
  #pragma unroll 1
  for (int idx = threadIdx.x; idx < R * E_virt; idx += blockDim.x) {
    const int s = idx / E_virt, e = idx - s * E_virt;
    const int* col = a.tile_hist + (size_t)s * a.tiles_per_src * E_virt + e;
    int acc = 0;
#pragma unroll 8
    for (int tb = 0; tb < a.tiles_per_src; ++tb) acc += __ldcg(col + (size_t)tb * E_virt);
    a.sps[idx] = acc;
    if (acc) {
      atomicAdd(&chunks[s * R + e / a.gpe], acc);
      atomicAdd(&s_splits[e], acc);
    }
  }
  #pragma unroll 1
  for (int i = threadIdx.x; i < R * ucw; i += blockDim.x) {
    const int s = i / ucw, d = i - s * ucw;
    const int* col = a.tile_uc + (size_t)s * a.tiles_per_src * ucw + d;
    int acc = 0;
#pragma unroll 8
    for (int tb = 0; tb < a.tiles_per_src; ++tb) acc += __ldcg(col + (size_t)tb * ucw);
    a.uc[i] = acc;
    s_uc[i] = acc;
  }
  __syncthreads();
  #pragma unroll 1
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) a.splits[e] = s_splits[e];
  __syncthreads();
  if (threadIdx.x == 0) ZEPP_FINE_MARK(a.status, TR_SCAN_COUNTS);
  // exclusive scan of splits -> expert_base (E_virt <= 4 * blockDim)
  {
    const int per = (E_virt + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * per;
    int local = 0;
    #pragma unroll 1
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) local += s_splits[lo + q];
    int total;
    int run = block_exclusive_scan(local, warp_tot, &total);
    #pragma unroll 1
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) { a.expert_base[lo + q] = run; s_base[lo + q] = run; run += s_splits[lo + q]; }
    if (threadIdx.x == 0) { a.expert_base[E_virt] = total; s_base[E_virt] = total; }
  }
  __syncthreads();
  if (threadIdx.x == 0) ZEPP_FINE_MARK(a.status, TR_SCAN_BASES);
  if (bases_in_place)
  #pragma unroll 1
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) {      // tile histograms -> tile bases, in place
    int run = s_base[e];
    #pragma unroll 1
    for (int b = 0; b < n_blocks; ++b) {
      const int h = a.tile_hist[(size_t)b * E_virt + e];
      a.tile_hist[(size_t)b * E_virt + e] = run;
      run += h;
    }
  }
  if (threadIdx.x == 0) {
    ZEPP_FINE_MARK(a.status, TR_SCAN_DEMANDS);
    long long out[8];
    demands_from_chunks(chunks, s_uc, R, a.L, a.relay_slots, a.direct, a.caps, out);
    #pragma unroll 1
    for (int i = 0; i < 8; ++i) a.demands[i] = out[i];
    viol = out[7];
    if (a.status) {
      a.status[ST_VIOLATION] = (unsigned long long)out[7];
      if (out[7]) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_CAPACITY);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) ZEPP_FINE_MARK(a.status, TR_SCAN_SCHED);
  // ---- this rank's GEMM schedule: token tiles of its groups in row order, one thread per group;
  //      groups marked as moved-in (bit 30 of their schedule word) go last (their weights land late)
  if (a.n_tiles != nullptr) {
    const int g0 = a.my_rank * a.gpe;
    const int m_start = s_base[g0];
    const int m_this = s_base[g0 + a.gpe] - m_start;
    const bool run_ok = viol == 0 && m_this <= a.recv_cap;
    const int e = threadIdx.x;                   // gpe <= blockDim.x
    int me = 0, late = 0;
    if (e >= 1 && e < a.gpe && run_ok) {
      me = s_splits[g0 + e];
      late = a.group_order != nullptr ? ((a.group_order[e] >> 30) & 1) : 0;
    }
    const int tile_rows = a.tile_rows_max > 0 ? a.tile_rows_max : kTileRowsMax;
    const int nt = (me + tile_rows - 1) / tile_rows;
    int tot_early, tot_late;
    const int pre_early = block_exclusive_scan(late ? 0 : nt, warp_tot, &tot_early);
    const int pre_late = block_exclusive_scan(late ? nt : 0, warp_tot, &tot_late);
    const int first = late ? tot_early + pre_late : pre_early;
    const int off = e < a.gpe ? s_base[g0 + (e < a.gpe ? e : 0)] - m_start : 0;
    #pragma unroll 1
    for (int t = 0; t < nt; ++t) {
      const int slot = first + t;
      if (slot < a.max_tiles) {
        a.tile_group[slot] = a.group_redirect != nullptr ? a.group_redirect[e] : e;
        a.tile_row0[slot] = off + t * tile_rows;
        a.tile_rows[slot] = min(tile_rows, me - t * tile_rows);
        a.tile_ready[slot] = 0u;
      }
    }
    if (threadIdx.x == 0) {
      trace_mark(a.status, TR_SCAN_END);
      a.m_this[0] = m_this;
      a.m_this[1] = m_start;
      *a.n_tiles = min(tot_early + tot_late, a.max_tiles);
    }
  }
  plan_heads(a, chunks, s_uc);
}

// Dispatch plan head and combine tables from the step's chunk table and unique counts.  Nothing
// on the GEMMs' path reads them: the layer computes them on request (plan_heads_kernel), the
// stand-alone metadata entry point inline.
__device__ void plan_heads(MetaArgs& a, const int* chunks, const int* s_uc) {
  const int R = a.R, NN = a.R / a.L, ucw = R + NN;
  // one warp each, lanes over destinations
  __shared__ long long seg_tab[132];
  const int lane_w = threadIdx.x & 31;
  if ((threadIdx.x >> 5) == 1 && a.dplan != nullptr) {
    // header + send segments + round-0 triples (python/zepp/routing.py:510-554, 613-623)
    const int W = R, L = a.L, rank = a.my_rank, me_n = rank / L, me_l = rank % L;
    const int nseg = L + NN - 1;
    long long err = 0, max_col = 0;
    #pragma unroll 1
    for (int d = lane_w; d < W; d += 32) {
      long long col = 0;
      #pragma unroll 1
      for (int s = 0; s < W; ++s) col += region_rows(s_uc, W, L, s, d);
      if (col > max_col) max_col = col;
    }
    #pragma unroll 1
    for (int i = lane_w; i < W * W; i += 32) {
      const int s = i / W, d = i - s * W;
      const long long cv = chunks[i];
      const long long uv = s_uc[s * ucw + d];
      if (!(uv >= 0 && uv <= cv && ((uv > 0) == (cv > 0)))) err |= 4;
      if (uv > s_uc[s * ucw + W + d / L]) err |= 8;
    }
    #pragma unroll 1
    for (int i = lane_w; i < W * NN; i += 32) {
      const int s = i / NN, n = i - s * NN;
      long long su = 0;
      #pragma unroll 1
      for (int l = 0; l < L; ++l) su += s_uc[s * ucw + n * L + l];
      if (s_uc[s * ucw + W + n] > su) err |= 8;
    }
    #pragma unroll 1
    for (int o = 16; o > 0; o >>= 1) {
      err |= __shfl_xor_sync(0xffffffffu, err, o);
      const long long m2 = __shfl_xor_sync(0xffffffffu, max_col, o);
      if (m2 > max_col) max_col = m2;
    }
    if (lane_w == 0) {
      long long seg = 0;
      int si = 0;
      seg_tab[0] = 0;
      #pragma unroll 1
      for (int n = 0; n < NN; ++n) {
        if (n == me_n) {
          #pragma unroll 1
          for (int dl = 0; dl < L; ++dl) { seg += s_uc[rank * ucw + n * L + dl]; seg_tab[++si] = seg; }
        } else {
          seg += s_uc[rank * ucw + W + n];
          seg_tab[++si] = seg;
        }
      }
    }
    __syncwarp();
    long long* P = a.dplan;
    #pragma unroll 1
    for (int i = lane_w; i <= nseg; i += 32) P[8 + i] = seg_tab[i];
    const int r0 = 8 + nseg + 1;
    #pragma unroll 1
    for (int dl = lane_w; dl < L; dl += 32) {
      const int d = me_n * L + dl;
      long long off = 0;
      #pragma unroll 1
      for (int s = 0; s < rank; ++s) off += region_rows(s_uc, W, L, s, d);
      P[r0 + 3 * dl + 0] = s_uc[rank * ucw + d];
      P[r0 + 3 * dl + 1] = seg_tab[me_n + dl];
      P[r0 + 3 * dl + 2] = off;
    }
    if (lane_w == 0) {
      if (max_col > a.caps[1]) err |= 16;
      if (seg_tab[nseg] > a.copies_per_rank) err |= 32;
      long long m0 = 0, off_me = 0;
      #pragma unroll 1
      for (int s = 0; s < W; ++s) m0 += chunks[s * W + rank];
      #pragma unroll 1
      for (int s = 0; s < rank; ++s) off_me += region_rows(s_uc, W, L, s, rank);
      P[0] = m0; P[1] = seg_tab[nseg]; P[2] = s_uc[rank * ucw + rank]; P[3] = seg_tab[me_n + me_l]; P[4] = off_me;
      P[5] = err; P[6] = 0; P[7] = 0;
    }
  }
  if ((threadIdx.x >> 5) == 2 && a.cplan != nullptr) {
    // combine tables on one node (python/zepp/routing.py:656-669): C[s][d] rows owner s returns to home d
    const int W = R, rank = a.my_rank;
    long long* so = a.cplan;
    long long* sr = so + W + 1;
    long long* dof = sr + W;
    long long* lo = dof + W;
    #pragma unroll 1
    for (int d = lane_w; d < W; d += 32) {
      sr[d] = chunks[d * W + rank];
      long long before = 0;
      #pragma unroll 1
      for (int s = 0; s < rank; ++s) before += chunks[d * W + s];
      dof[d] = before;
    }
    if (lane_w == 0) {
      long long acc = 0;
      so[0] = 0;
      #pragma unroll 1
      for (int d = 0; d < W; ++d) { acc += chunks[d * W + rank]; so[d + 1] = acc; }
    }
    if (lane_w == 1) {
      long long acc = 0;
      lo[0] = 0;
      #pragma unroll 1
      for (int s = 0; s < W; ++s) { acc += chunks[rank * W + s]; lo[s + 1] = acc; }
    }
  }
}

// sps / uc of the last step -> plan heads (one block; run on request, off the step's path)
__global__ void __launch_bounds__(128) plan_heads_kernel(MetaArgs a) {
  extern __shared__ int sm[];
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, ucw = R + NN;
  int* chunks = sm;
  int* s_uc = sm + R * R;
  for (int i = threadIdx.x; i < R * R; i += blockDim.x) {
    const int s = i / R, d = i - s * R;
    int acc = 0;
    for (int e = 0; e < a.gpe; ++e) acc += a.sps[s * E_virt + d * a.gpe + e];
    chunks[i] = acc;
  }
  for (int i = threadIdx.x; i < R * ucw; i += blockDim.x) s_uc[i] = a.uc[i];
  __syncthreads();
  plan_heads(a, chunks, s_uc);
}

__global__ void __launch_bounds__(kMetaThreads) meta_pass2_kernel(MetaArgs a) {
  extern __shared__ int sm[];
  const int E_virt = a.R * a.gpe, SK = a.S * a.K;
  const int src = blockIdx.x / a.tiles_per_src;
  const int tb = blockIdx.x - src * a.tiles_per_src;
  const int* tbase = a.tile_hist + (size_t)blockIdx.x * E_virt;
  const int T = a.tokens_per_tile * a.K;
  const int n_warps = (T + 31) / 32;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a.status, TR_PASS2);
  int* wc = sm;                           // [n_warps][E_virt] copies of expert e in warp w, then their base
  for (int i = threadIdx.x; i < n_warps * E_virt; i += blockDim.x) wc[i] = 0;
  __syncthreads();
  const int n = tb * T + threadIdx.x;
  const bool valid = threadIdx.x < T && n < SK;
  const size_t flat = (size_t)src * SK + (valid ? n : 0);
  int e = valid ? a.vce[flat] : -1;
  const bool pad = valid && e < 0;
  if (e < 0) e = -1 - (int)(threadIdx.x & 31);                          // invalid lanes and pad copies never match
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  unsigned m = 0;
  if (wid < n_warps) {
    m = __match_any_sync(0xffffffffu, e);
    if (valid && !pad && lane == __ffs(m) - 1) wc[wid * E_virt + e] = __popc(m);
  }
  __syncthreads();
  for (int x = threadIdx.x; x < E_virt; x += blockDim.x) {      // exclusive prefix over the tile's warps
    int run = tbase[x];
    for (int w = 0; w < n_warps; ++w) {
      const int c = wc[w * E_virt + x];
      wc[w * E_virt + x] = run;
      run += c;
    }
  }
  __syncthreads();
  // staged dispatch: the source stored each token once per destination rank at slot = number of its
  // earlier tokens that also go to that rank; the same slot follows here from the per-tile unique
  // counts (tiles hold whole tokens) and a scan over the tile's tokens
  __shared__ int s_tokslot[kMetaThreads];
  __shared__ int s_warp_tot[33];
  if (a.staged && a.row_tok != nullptr) {
    const int tpt = a.tokens_per_tile;
    for (int t = threadIdx.x; t < tpt; t += blockDim.x) s_tokslot[t] = 0;
    __syncthreads();
    if (valid && !pad && e / a.gpe == a.my_rank) s_tokslot[threadIdx.x / a.K] = 1;
    __syncthreads();
    const int f = threadIdx.x < tpt ? s_tokslot[threadIdx.x] : 0;
    int total;
    int pre = block_exclusive_scan(f, s_warp_tot, &total);
    const int ucw = a.R + a.R / a.L;
    for (int q = 0; q < tb; ++q) pre += a.tile_uc[(size_t)(src * a.tiles_per_src + q) * ucw + a.my_rank];
    __syncthreads();
    if (threadIdx.x < tpt) s_tokslot[threadIdx.x] = pre;
    __syncthreads();
  }
  if (!valid) return;
  if (pad) { a.scatter_index[flat] = -1; return; }
  const int idx = wc[wid * E_virt + e] + __popc(m & ((1u << lane) - 1u));
  a.scatter_index[flat] = idx;
  if (a.row_tok != nullptr && e / a.gpe == a.my_rank) {
    const int r = idx - a.m_this[1];
    if (r >= 0 && r < a.recv_cap) {
      a.row_tok[r] = src * a.S + (a.staged ? s_tokslot[threadIdx.x / a.K] : n / a.K);
      a.row_scale[r] = a.probs_all ? a.probs_all[flat] : 1.0f;
      a.row_dst[r] = ((long long)src << 40) | ((long long)n * a.hidden);
    }
  }
}

// Shared memory of the fused kernel (ints): the larger of a tile block's tables
// (hist[E] | ucs[R+NN] | tot[E] | base[E+1] | v[threads] | wc[max(warps, 16) * E]) and the tables block's scan.
__host__ __device__ inline size_t meta_fused_smem_ints(int R, int NN, int E_virt, int tokens_per_tile, int K) {
  const int n_warps = (tokens_per_tile * K + 31) / 32;
  const size_t tile = 3 * (size_t)E_virt + (size_t)(R + NN) + 1 + kMetaThreads + (size_t)(n_warps > 16 ? n_warps : 16) * E_virt;
  const size_t scan = meta_scan_smem_ints(R, NN, E_virt);
  return tile > scan ? tile : scan;
}

}  // namespace zepp
