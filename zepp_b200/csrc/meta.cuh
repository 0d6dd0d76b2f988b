// Routed metadata of a step: virtual group ids, per-expert counts, the deterministic stable
// scatter index, per-source splits, unique (token, destination) counts, exact buffer demands with
// their violation mask, the dispatch / combine plan heads, and the row / tile tables the two GEMM
// kernels read.  Replaces DispatchGemmOp::derive_routed_meta (src/dispatch/ths_op/dispatch_gemm.cc:916-1101;
// kernels src/dispatch/sort_util.cu:354-541, 957-1122, 1153-1500), planner_tail_kernel
// (src/planner/lane_device.cu:526-540) and the combine tables (src/combine/combine_kernels.cu:1308,1546);
// host references python/zepp/routing.py:306-331, python/zepp/capacity.py:30-55.
//
// Three launches, no atomics on global memory, no host read:
//   pass1  one block per tile of one source's entries: vce / probs_all (from the gathered routing
//          rows), per-tile expert histogram, per-tile unique owner / node counts;
//   scan   one block: splits, sps, uc, exclusive bases (tile histograms become tile bases in
//          place), demands + mask, plan heads, this rank's tile schedule;
//   pass2  same grid as pass1: stable rank of every copy inside its expert (warps of a tile take
//          turns, lanes rank themselves with match_any), scatter_index, and for copies owned by
//          this rank the GEMM row tables (source token, home slot, top-k weight).
#pragma once
#include "common.cuh"
#include "planner.cuh"

namespace zepp {

constexpr int kMetaThreads = 1024;
constexpr int kTileRowsMax = 128;

struct MetaArgs {
  // input: either the gathered routing rows [R, 2*SK] (phys | weight bits) or vce directly
  const int* gathered;
  const int* vce_in;
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
  const int* group_order;   // [gpe] schedule word per group (bit 30 = moved-in slot: its tiles go last) or nullptr
  // exchange wait
  const unsigned long long* routing_flags;
  unsigned long long epoch, limit_ns;
  unsigned long long* status;
};

__global__ void __launch_bounds__(kMetaThreads) meta_pass1_kernel(MetaArgs a) {
  extern __shared__ int sm[];
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, SK = a.S * a.K;
  int* hist = sm;                       // [E_virt]
  int* ucs = sm + E_virt;               // [R + NN]
  if (!block_wait_all(a.routing_flags, R, a.epoch, a.limit_ns, a.status, WAIT_ROUTING)) return;
  const int src = blockIdx.x / a.tiles_per_src;
  const int tb = blockIdx.x - src * a.tiles_per_src;
  for (int i = threadIdx.x; i < E_virt + R + NN; i += blockDim.x) sm[i] = 0;
  __syncthreads();
  const int T = a.tokens_per_tile * a.K;
  const int n_lo = tb * T;
  const int n_hi = min(SK, n_lo + T);
  for (int n = n_lo + threadIdx.x; n < n_hi; n += blockDim.x) {
    int v;
    const size_t flat = (size_t)src * SK + n;
    if (a.gathered) {
      const int phys = a.gathered[(size_t)src * 2 * SK + n];
      v = (phys / a.nlp) * a.gpe + 1 + phys % a.nlp;
      a.probs_all[flat] = __int_as_float(a.gathered[(size_t)src * 2 * SK + SK + n]);
    } else {
      v = a.vce_in[flat];
    }
    if (v < 0 || v >= E_virt) {
      if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
      v = 0;
    }
    a.vce[flat] = v;
    atomicAdd(&hist[v], 1);
  }
  __syncthreads();
  // unique owners / nodes per token (a token may pick one rank several times)
  const int t_lo = tb * a.tokens_per_tile;
  const int t_hi = min(a.S, t_lo + a.tokens_per_tile);
  for (int t = t_lo + threadIdx.x; t < t_hi; t += blockDim.x) {
    unsigned long long owners = 0, nodes = 0;
    for (int k = 0; k < a.K; ++k) {
      const int o = a.vce[((size_t)src * a.S + t) * a.K + k] / a.gpe;
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
}

// Exact demands of a step (python/zepp/capacity.py:30-55) by one thread; R <= 64.
__device__ void demands_serial(const int* sps, const int* uc, int W, int L, int gpe, int relay_slots, int direct,
                               const long long* caps, long long* out) {
  const int NN = W / L, E_virt = W * gpe;
  long long recv_rows = 0, pair = 0;
  for (int d = 0; d < W; ++d) {
    long long col = 0;
    for (int s = 0; s < W; ++s) {
      long long ch = 0;
      for (int e = 0; e < gpe; ++e) ch += sps[s * E_virt + d * gpe + e];
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
          for (int ls = 0; ls < L; ++ls)
            for (int e = 0; e < gpe; ++e) cv += sps[(ns * L + k) * E_virt + (n * L + ls) * gpe + e];
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
    const int ci[7] = {0, 1, 2, 3, 4, 5, 6};
    for (int b = 0; b < 7; ++b)
      if (dem[di[b]] > caps[ci[b]]) mask |= 1ll << b;
  }
  out[7] = mask;
}

__device__ __forceinline__ long long region_rows(const int* uc, int W, int L, int s, int d) {
  const int NN = W / L;
  return (s / L == d / L) ? uc[s * (W + NN) + d] : uc[s * (W + NN) + W + d / L];
}

__global__ void __launch_bounds__(kMetaThreads) meta_scan_kernel(MetaArgs a) {
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, ucw = R + NN;
  const int n_blocks = R * a.tiles_per_src;
  __shared__ int warp_tot[32];
  __shared__ long long viol;
  // per source splits, totals, tile bases (in place)
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) {
    int tot = 0;
    for (int s = 0; s < R; ++s) {
      int acc = 0;
      for (int tb = 0; tb < a.tiles_per_src; ++tb) acc += a.tile_hist[(size_t)(s * a.tiles_per_src + tb) * E_virt + e];
      a.sps[s * E_virt + e] = acc;
      tot += acc;
    }
    a.splits[e] = tot;
  }
  for (int i = threadIdx.x; i < R * ucw; i += blockDim.x) {
    const int s = i / ucw, d = i - s * ucw;
    int acc = 0;
    for (int tb = 0; tb < a.tiles_per_src; ++tb) acc += a.tile_uc[(size_t)(s * a.tiles_per_src + tb) * ucw + d];
    a.uc[i] = acc;
  }
  __syncthreads();
  // exclusive scan of splits -> expert_base (E_virt <= 4 * blockDim)
  {
    const int per = (E_virt + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * per;
    int local = 0;
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) local += a.splits[lo + q];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int incl = local;
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      int v = lane < (int)(blockDim.x >> 5) ? warp_tot[lane] : 0;
      int inc2 = v;
      for (int off = 1; off < 32; off <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, inc2, off);
        if (lane >= off) inc2 += u;
      }
      warp_tot[lane] = inc2 - v;
    }
    __syncthreads();
    int run = warp_tot[wid] + incl - local;
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) { a.expert_base[lo + q] = run; run += a.splits[lo + q]; }
    if (threadIdx.x == blockDim.x - 1) a.expert_base[E_virt] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) {
    int run = a.expert_base[e];
    for (int b = 0; b < n_blocks; ++b) {
      const int h = a.tile_hist[(size_t)b * E_virt + e];
      a.tile_hist[(size_t)b * E_virt + e] = run;
      run += h;
    }
  }
  if (threadIdx.x == 0) {
    long long out[8];
    demands_serial(a.sps, a.uc, R, a.L, a.gpe, a.relay_slots, a.direct, a.caps, out);
    for (int i = 0; i < 8; ++i) a.demands[i] = out[i];
    viol = out[7];
    if (a.status) {
      a.status[ST_VIOLATION] = (unsigned long long)out[7];
      if (out[7]) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_CAPACITY);
    }
  }
  __syncthreads();
  // ---- this rank's GEMM schedule: token tiles of its groups in row order; groups marked as
  //      moved-in (bit 30 of their schedule word) are placed last (their weights land late)
  if (threadIdx.x == 0 && a.n_tiles != nullptr) {
    const int g0 = a.my_rank * a.gpe;
    const int m_start = a.expert_base[g0];
    const int m_this = a.expert_base[g0 + a.gpe] - m_start;
    a.m_this[0] = m_this;
    a.m_this[1] = m_start;
    int nt = 0;
    if (viol == 0 && m_this <= a.recv_cap) {
      for (int pass = 0; pass < 2; ++pass) {
        for (int e = 1; e < a.gpe; ++e) {
          const bool late = a.group_order != nullptr && ((a.group_order[e] >> 30) & 1);
          if ((pass == 1) != late) continue;
          const int me = a.splits[g0 + e];
          const int off = a.expert_base[g0 + e] - m_start;
          for (int r = 0; r < me && nt < a.max_tiles; r += kTileRowsMax) {
            a.tile_group[nt] = e;
            a.tile_row0[nt] = off + r;
            a.tile_rows[nt] = min(kTileRowsMax, me - r);
            a.tile_ready[nt] = 0u;
            ++nt;
          }
        }
      }
    }
    *a.n_tiles = nt;
  }
  // ---- plan heads
  if (threadIdx.x == 32 && a.dplan != nullptr) {
    // header + send segments + round-0 triples (python/zepp/routing.py:510-554, 613-623)
    const int W = R, L = a.L, rank = a.my_rank, me_n = rank / L, me_l = rank % L;
    const int nseg = L + NN - 1;
    long long err = 0;
    long long max_col = 0;
    for (int d = 0; d < W; ++d) {
      long long col = 0;
      for (int s = 0; s < W; ++s) col += region_rows(a.uc, W, L, s, d);
      if (col > max_col) max_col = col;
    }
    for (int s = 0; s < W; ++s) {
      for (int d = 0; d < W; ++d) {
        long long cv = 0;
        for (int e = 0; e < a.gpe; ++e) cv += a.sps[s * E_virt + d * a.gpe + e];
        const long long uv = a.uc[s * ucw + d];
        if (!(uv >= 0 && uv <= cv && ((uv > 0) == (cv > 0)))) err |= 4;
        if (uv > a.uc[s * ucw + W + d / L]) err |= 8;
      }
      for (int n = 0; n < NN; ++n) {
        long long su = 0;
        for (int l = 0; l < L; ++l) su += a.uc[s * ucw + n * L + l];
        if (a.uc[s * ucw + W + n] > su) err |= 8;
      }
    }
    long long* P = a.dplan;
    long long seg = 0;
    int si = 0;
    P[8 + 0] = 0;
    long long seg_me = 0, seg_tab[128];
    seg_tab[0] = 0;
    for (int n = 0; n < NN; ++n) {
      if (n == me_n) {
        for (int dl = 0; dl < L; ++dl) { seg += a.uc[rank * ucw + n * L + dl]; seg_tab[++si] = seg; }
      } else {
        seg += a.uc[rank * ucw + W + n];
        seg_tab[++si] = seg;
      }
    }
    for (int i = 0; i <= nseg; ++i) P[8 + i] = seg_tab[i];
    const int r0 = 8 + nseg + 1;
    for (int dl = 0; dl < L; ++dl) {
      const int d = me_n * L + dl;
      long long off = 0;
      for (int s = 0; s < rank; ++s) off += region_rows(a.uc, W, L, s, d);
      P[r0 + 3 * dl + 0] = a.uc[rank * ucw + d];
      P[r0 + 3 * dl + 1] = seg_tab[me_n + dl];
      P[r0 + 3 * dl + 2] = off;
    }
    if (max_col > a.caps[1]) err |= 16;
    if (seg_tab[nseg] > a.copies_per_rank) err |= 32;
    long long m0 = 0;
    for (int s = 0; s < W; ++s)
      for (int e = 0; e < a.gpe; ++e) m0 += a.sps[s * E_virt + rank * a.gpe + e];
    long long off_me = 0;
    for (int s = 0; s < rank; ++s) off_me += region_rows(a.uc, W, L, s, rank);
    seg_me = seg_tab[me_n + me_l];
    P[0] = m0; P[1] = seg_tab[nseg]; P[2] = a.uc[rank * ucw + rank]; P[3] = seg_me; P[4] = off_me; P[5] = err;
    P[6] = 0; P[7] = 0;
  }
  if (threadIdx.x == 64 && a.cplan != nullptr) {
    // combine tables on one node (python/zepp/routing.py:656-669): C[s][d] rows owner s returns to home d
    const int W = R, rank = a.my_rank;
    long long* so = a.cplan;
    long long* sr = so + W + 1;
    long long* dof = sr + W;
    long long* lo = dof + W;
    long long acc = 0;
    so[0] = 0;
    for (int d = 0; d < W; ++d) {
      long long c = 0;
      for (int e = 0; e < a.gpe; ++e) c += a.sps[d * E_virt + rank * a.gpe + e];
      sr[d] = c;
      acc += c;
      so[d + 1] = acc;
      long long before = 0;
      for (int s = 0; s < rank; ++s)
        for (int e = 0; e < a.gpe; ++e) before += a.sps[d * E_virt + s * a.gpe + e];
      dof[d] = before;
    }
    acc = 0;
    lo[0] = 0;
    for (int s = 0; s < W; ++s) {
      long long c = 0;
      for (int e = 0; e < a.gpe; ++e) c += a.sps[rank * E_virt + s * a.gpe + e];
      acc += c;
      lo[s + 1] = acc;
    }
  }
}

__global__ void __launch_bounds__(kMetaThreads) meta_pass2_kernel(MetaArgs a) {
  extern __shared__ int sm[];
  const int E_virt = a.R * a.gpe, SK = a.S * a.K;
  int* cnt = sm;                          // running position per expert inside this tile
  const int src = blockIdx.x / a.tiles_per_src;
  const int tb = blockIdx.x - src * a.tiles_per_src;
  const int* tbase = a.tile_hist + (size_t)blockIdx.x * E_virt;
  for (int e = threadIdx.x; e < E_virt; e += blockDim.x) cnt[e] = tbase[e];
  __syncthreads();
  const int T = a.tokens_per_tile * a.K;
  const int n = tb * T + threadIdx.x;
  const bool valid = threadIdx.x < T && n < SK;
  const size_t flat = (size_t)src * SK + (valid ? n : 0);
  const int e = valid ? a.vce[flat] : -1 - (int)(threadIdx.x & 31);     // invalid lanes never match
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int n_warps = (T + 31) / 32;
  int idx = -1;
  for (int w = 0; w < n_warps; ++w) {
    if (wid == w) {
      const unsigned m = __match_any_sync(0xffffffffu, e);
      const int leader = __ffs(m) - 1;
      int off = 0;
      if (valid && lane == leader) { off = cnt[e]; cnt[e] = off + __popc(m); }
      off = __shfl_sync(0xffffffffu, off, leader);
      idx = off + __popc(m & ((1u << lane) - 1u));
    }
    __syncthreads();
  }
  if (!valid) return;
  a.scatter_index[flat] = idx;
  if (a.row_tok != nullptr && e / a.gpe == a.my_rank) {
    const int r = idx - a.m_this[1];
    if (r >= 0 && r < a.recv_cap) {
      a.row_tok[r] = src * a.S + n / a.K;
      a.row_scale[r] = a.probs_all ? a.probs_all[flat] : 1.0f;
      a.row_dst[r] = ((long long)src << 40) | ((long long)n * a.hidden);
    }
  }
}

}  // namespace zepp
