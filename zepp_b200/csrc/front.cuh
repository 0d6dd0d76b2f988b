// The front end of a layer step as ONE cooperative launch: routed metadata (count -> grid barrier -> rank, plus a
// block that writes the step's tables) and, beside it in the same grid, the blocks that have nothing to wait
// for: the single-replica routing with its exchange (route blocks) and the staged dispatch push of this rank's
// token rows (push blocks).  The metadata blocks wait for every rank's routing rows -- this rank's own come from
// the route blocks of the same launch, which is safe because a cooperative launch keeps every block resident --
// while the NVLink transfer of the token rows runs under them.
//   tile blocks    [0, R * tiles_per_src)   one tile of one source's entries each
//   tables block   the next one             splits, sps, uc, bases, demands, plan heads, this rank's tile schedule
//   route blocks   the next n_route         python/zepp/planner.py:122 (send row) for single-replica placements
//   push blocks    the last n_push          src/dwire/dispatch_wire.cu:107-210 (dedup'ed pack-push)
// Replaces, in one launch, planner_tail + derive_routed_meta + the dispatch wire's push of the reference
// (src/planner/lane_device.cu:526-540, src/dispatch/ths_op/dispatch_gemm.cc:916-1101).
#pragma once
#include "layer_kernels.cuh"
#include "meta.cuh"

namespace zepp {

struct FrontArgs {
  int n_route, n_push;     // blocks of each optional role (0: the role runs elsewhere or not at all)
  int first;               // this launch is the step's first kernel: it works under *ctr + 1 and commits it
  unsigned int* route_counter;   // self-resetting arrival counter of the route blocks
  SimpleRouteArgs route;
  PushArgs push;
};

__global__ void __launch_bounds__(kMetaThreads) meta_fused_kernel(MetaArgs a, const FrontArgs f) {
  extern __shared__ int sm[];
  const int R = a.R, NN = a.R / a.L, E_virt = a.R * a.gpe, SK = a.S * a.K, ucw = R + NN;
  const int n_tile_blocks = R * a.tiles_per_src;
  const bool tables_block = (int)blockIdx.x == n_tile_blocks;
  int* hist = sm;                          // [E_virt] this tile's counts, later its bases
  int* ucs = hist + E_virt;                // [R + NN]
  int* s_tot = ucs + ucw;                  // [E_virt] copies per virtual expert
  int* s_base = s_tot + E_virt;            // [E_virt + 1] exclusive bases
  int* s_v = s_base + E_virt + 1;          // [threads] vce of this tile's entries
  int* wc = s_v + kMetaThreads;            // [warps][E_virt]; first used for partial sums
  __shared__ int s_go;
  __shared__ int s_tokslot[kMetaThreads];
  __shared__ int s_warp_tot[33];
  const bool local = a.local_topk != nullptr;
  const bool first = local || f.first != 0;
  const unsigned long long epoch = step_epoch(a.epoch_ptr, first);
  if (a.epoch_ptr != nullptr && (epoch & 1)) { a.gathered = a.gathered_odd; a.gathered_out = a.gathered_out_odd; }
  // generation of the grid barrier, read before this block can have arrived
  const unsigned int gen0 = threadIdx.x == 0 ? ld_acquire_gpu_u32(a.grid_sync + 1) : 0u;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (first || f.n_route > 0) {
      trace_mark(a.status, TR_ROUTE);
      trace_mark(a.status, TR_RING + (int)(epoch & 15));
    }
    trace_mark(a.status, TR_PASS1);
  }
  if ((int)blockIdx.x > n_tile_blocks) {
    // ---- route / push blocks: arrive at the grid barrier at once (they have read the epoch), never wait at it
    if (threadIdx.x == 0 && atomicInc(a.grid_sync, gridDim.x - 1) == gridDim.x - 1) {
      __threadfence();
      atomicExch(a.grid_sync + 1, gen0 + 1u);
    }
    const int role = (int)blockIdx.x - n_tile_blocks - 1;
    if (role < f.n_route) {
      #pragma unroll 1
      for (int g = threadIdx.x; g < f.route.G; g += blockDim.x) sm[g] = f.route.slot_of[g];
      __syncthreads();
      route_simple_rows(f.route, sm, role, f.n_route, epoch);
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicInc(f.route_counter, f.n_route - 1) == (unsigned int)f.n_route - 1) {
          __threadfence_system();
          #pragma unroll 1
          for (int p = 0; p < f.route.world; ++p)
            st_relaxed_sys(reinterpret_cast<unsigned long long*>(f.route.flags.ptr[p]) + f.route.my_rank, epoch);
        }
      }
    } else {
      // The routing rows are small and every rank's metadata waits for them: the token rows (megabytes on the
      // same links) follow them, so a push block starts once this rank's route blocks have raised their flag here.
      if (f.n_route > 0 && threadIdx.x == 0) {
        const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(f.route.flags.ptr[f.route.my_rank]) + f.route.my_rank;
        if (!wait_epoch_geq(mine, epoch, a.limit_ns != 0 ? a.limit_ns : 4000000000ull))
          record_timeout(a.status, WAIT_ROUTING, f.route.my_rank, (long long)epoch);      // push anyway: the rows are still needed
      }
      __syncthreads();
      push_block(f.push, role - f.n_route, f.n_push, epoch);
    }
    return;
  }
  if (!block_wait_all(a.routing_flags, R, epoch, a.limit_ns, a.status, WAIT_ROUTING)) return;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a.status, TR_PASS1_GO);
  const int src = tables_block ? 0 : blockIdx.x / a.tiles_per_src;
  const int tb = tables_block ? 0 : blockIdx.x - src * a.tiles_per_src;
  const int T = a.tokens_per_tile * a.K;                 // entries of a tile (<= threads: one per thread)
  const int n = tb * T + threadIdx.x;
  const bool valid = !tables_block && (int)threadIdx.x < T && n < SK;
  const size_t flat = (size_t)src * SK + (valid ? n : 0);
  int my_v = -1;
  // ---- count
  if (!tables_block) {
    #pragma unroll 1
    for (int i = threadIdx.x; i < E_virt + ucw; i += blockDim.x) sm[i] = 0;
    __syncthreads();
    if (valid) {
      my_v = meta_decode_entry(a, local, src, n, SK, E_virt);
      if (my_v >= 0) atomicAdd(&hist[my_v], 1);
    }
    s_v[threadIdx.x] = my_v;
    __syncthreads();
    const int t_lo = tb * a.tokens_per_tile;
    const int t_cnt = min(a.S, t_lo + a.tokens_per_tile) - t_lo;
    if ((int)threadIdx.x < t_cnt) {
      unsigned long long owners = 0, nodes = 0;
      #pragma unroll 1
      for (int k = 0; k < a.K; ++k) {
        const int v = s_v[threadIdx.x * a.K + k];
        if (v < 0) continue;
        const int o = v / a.gpe;
        owners |= 1ull << o;
        nodes |= 1ull << (o / a.L);
      }
      while (owners) { const int o = __ffsll((long long)owners) - 1; owners &= owners - 1; atomicAdd(&ucs[o], 1); }
      while (nodes) { const int o = __ffsll((long long)nodes) - 1; nodes &= nodes - 1; atomicAdd(&ucs[R + o], 1); }
    }
    __syncthreads();
    int* th = a.tile_hist + (size_t)blockIdx.x * E_virt;
    #pragma unroll 1
    for (int e = threadIdx.x; e < E_virt; e += blockDim.x) th[e] = hist[e];
    int* tu = a.tile_uc + (size_t)blockIdx.x * ucw;
    #pragma unroll 1
    for (int i = threadIdx.x; i < ucw; i += blockDim.x) tu[i] = ucs[i];
  }
  // ---- grid barrier (every block of a cooperative launch is resident; the wait is bounded all the same)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int go = 1;
    if (atomicInc(a.grid_sync, gridDim.x - 1) == gridDim.x - 1) {
      __threadfence();
      atomicExch(a.grid_sync + 1, gen0 + 1u);
    } else {
      const unsigned long long t0 = globaltimer_ns();
      const unsigned long long limit = a.limit_ns != 0 ? a.limit_ns : 4000000000ull;
      while (ld_acquire_gpu_u32(a.grid_sync + 1) == gen0) {
        if (globaltimer_ns() - t0 > limit) {
          record_timeout(a.status, WAIT_BARRIER, blockIdx.x, (long long)epoch);
          go = 0;
          break;
        }
      }
    }
    s_go = go;
  }
  __syncthreads();
  if (!s_go) return;
  if (tables_block) {
    // ---- scan: the step's tables (the tile blocks never wait for them)
    meta_scan_body(a, sm, false);
    // every block read the counter before it arrived at the barrier
    if (first && threadIdx.x == 0 && a.epoch_ptr != nullptr) *const_cast<unsigned long long*>(a.epoch_ptr) = epoch;
    return;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a.status, TR_PASS2);
  // ---- this tile's bases: copies of every expert in all tiles (-> exclusive bases) and in the tiles before this one
  {
    int P = (int)blockDim.x / E_virt;
    P = P < 1 ? 1 : (P > 8 ? 8 : P);
    const int chunk = (n_tile_blocks + P - 1) / P;
    int* p_tot = wc;
    int* p_bef = wc + P * E_virt;
    #pragma unroll 1
    for (int idx = threadIdx.x; idx < P * E_virt; idx += blockDim.x) {
      const int sl = idx / E_virt, e = idx - sl * E_virt;
      const int b_lo = sl * chunk, b_hi = min(n_tile_blocks, b_lo + chunk);
      int t = 0, b4 = 0;
      #pragma unroll 4
      for (int b = b_lo; b < b_hi; ++b) {
        const int h = __ldcg(a.tile_hist + (size_t)b * E_virt + e);
        t += h;
        if (b < (int)blockIdx.x) b4 += h;
      }
      p_tot[idx] = t;
      p_bef[idx] = b4;
    }
    __syncthreads();
    #pragma unroll 1
    for (int e = threadIdx.x; e < E_virt; e += blockDim.x) {
      int t = 0, b4 = 0;
      #pragma unroll 1
      for (int sl = 0; sl < P; ++sl) { t += p_tot[sl * E_virt + e]; b4 += p_bef[sl * E_virt + e]; }
      s_tot[e] = t;
      hist[e] = b4;
    }
    __syncthreads();
    const int per = (E_virt + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * per;
    int mine = 0;
    #pragma unroll 1
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) mine += s_tot[lo + q];
    int total;
    int run = block_exclusive_scan(mine, s_warp_tot, &total);
    #pragma unroll 1
    for (int q = 0; q < per; ++q)
      if (lo + q < E_virt) { s_base[lo + q] = run; run += s_tot[lo + q]; }
    if (threadIdx.x == 0) s_base[E_virt] = total;
    __syncthreads();
    #pragma unroll 1
    for (int e = threadIdx.x; e < E_virt; e += blockDim.x) hist[e] += s_base[e];
  }
  // ---- rank: stable position of every copy inside its expert
  const int n_warps = (T + 31) / 32;
  #pragma unroll 1
  for (int i = threadIdx.x; i < n_warps * E_virt; i += blockDim.x) wc[i] = 0;
  __syncthreads();
  const bool pad = valid && my_v < 0;
  const int e = my_v >= 0 ? my_v : -1 - (int)(threadIdx.x & 31);        // invalid lanes and pad copies never match
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  unsigned m = 0;
  if (wid < n_warps) {
    m = __match_any_sync(0xffffffffu, e);
    if (my_v >= 0 && lane == __ffs(m) - 1) wc[wid * E_virt + e] = __popc(m);
  }
  __syncthreads();
  #pragma unroll 1
  for (int x = threadIdx.x; x < E_virt; x += blockDim.x) {      // exclusive prefix over the tile's warps
    int run = hist[x];
    #pragma unroll 1
    for (int w = 0; w < n_warps; ++w) {
      const int c = wc[w * E_virt + x];
      wc[w * E_virt + x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (a.staged && a.row_tok != nullptr) {
    // staging slot of a token on this rank = number of earlier tokens of its source that also come here
    const int tpt = a.tokens_per_tile;
    #pragma unroll 1
    for (int t = threadIdx.x; t < tpt; t += blockDim.x) s_tokslot[t] = 0;
    __syncthreads();
    if (my_v >= 0 && my_v / a.gpe == a.my_rank) s_tokslot[threadIdx.x / a.K] = 1;
    __syncthreads();
    const int f = (int)threadIdx.x < tpt ? s_tokslot[threadIdx.x] : 0;
    int total;
    int pre = block_exclusive_scan(f, s_warp_tot, &total);
    if (wid == 0) {                      // tokens of the source's earlier tiles that come here
      int acc = 0;
      #pragma unroll 4
      for (int q = lane; q < tb; q += 32) acc += __ldcg(a.tile_uc + (size_t)(src * a.tiles_per_src + q) * ucw + a.my_rank);
      #pragma unroll 1
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_go = acc;
    }
    __syncthreads();
    if ((int)threadIdx.x < tpt) s_tokslot[threadIdx.x] = pre + s_go;
    __syncthreads();
  }
  if (!valid) return;
  if (pad) { a.scatter_index[flat] = -1; return; }
  const int idx = wc[wid * E_virt + e] + __popc(m & ((1u << lane) - 1u));
  a.scatter_index[flat] = idx;
  if (a.row_tok != nullptr && e / a.gpe == a.my_rank) {
    const int r = idx - s_base[a.my_rank * a.gpe];
    if (r >= 0 && r < a.recv_cap) {
      a.row_tok[r] = src * a.S + (a.staged ? s_tokslot[threadIdx.x / a.K] : n / a.K);
      a.row_scale[r] = a.probs_all ? a.probs_all[flat] : 1.0f;
      a.row_dst[r] = ((long long)src << 40) | ((long long)n * a.hidden);
    }
  }
}

}  // namespace zepp
