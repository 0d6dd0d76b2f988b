// Integer planning kernels: per-expert demand histogram + exchange, capacity-constrained replica
// routing (rotation water-fill, budgets, deterministic ordinal assignment, per-token vacate) and
// the routing exchange.  All results are pure integer functions of replicated inputs, so every
// rank derives identical tables; they are bit-exact against the reference's host planner
// (python/zepp/routing.py), not against its device router, whose per-entry assignment uses
// relaxed atomic tickets (src/planner/routing.cu:247,448).
#pragma once
#include "common.cuh"

namespace zepp {

constexpr int kMaxRep = 32;      // replicas of one expert the tables hold (reference: K_MAX_REP)
constexpr int kMaxRanks = 64;

__host__ __device__ inline int route_cm(int R) { return R < kMaxRep ? R : kMaxRep; }

// Route workspace layout (int32 words).
struct RouteWs {
  int rep, rphys, c, D, U, Lb, fill, M, rel, ext, total;
};
__host__ __device__ inline RouteWs route_ws_layout(int G, int R) {
  const int CM = route_cm(R);
  RouteWs w;
  int o = 0;
  w.rep = o;   o += G * CM;        // host rank of replica jj (ascending), -1 pad
  w.rphys = o; o += G * CM;        // physical slot of replica jj
  w.c = o;     o += G;             // replica count
  w.D = o;     o += G;             // global demand
  w.U = o;     o += G;             // upper bound per replica
  w.Lb = o;    o += G;             // lower bound per replica
  w.fill = o;  o += G * CM;        // rows on replica jj after the water-fill
  w.M = o;     o += G * R * CM;    // takes M[g][i][jj]
  w.rel = o;   o += G * CM;        // release budget of this source
  w.ext = o;   o += G * CM;        // extra budget of this source
  w.total = o;
  return w;
}

struct PeerTable {
  void* ptr[kMaxRanks];
};

// Step epoch.  A layer keeps a device-resident step counter so that a whole step can be replayed
// as a CUDA graph with unchanged kernel arguments.  The first kernel of a step works under epoch
// *ctr + 1 and its last block commits it; every later kernel of the step reads *ctr.  Buffers that
// are double-buffered by step parity are passed as pairs and selected with (epoch & 1).
__device__ __forceinline__ unsigned long long step_epoch(const unsigned long long* ctr, bool first) {
  if (ctr == nullptr) return 0ull;
  const unsigned long long v = *reinterpret_cast<const volatile unsigned long long*>(ctr);
  return first ? v + 1 : v;
}

// ---------------------------------------------------------------------------------------
// loads: d_own[G] = bincount(topk_own) and its publication to every rank
// (python/zepp/planner.py:104-112: index_add_ + all_gather_into_tensor).
// One block.  dst.ptr[p] is rank p's loads table [R, G]; flags.ptr[p] its arrival words [R].
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void loads_publish_block(const int* __restrict__ topk_own, int n_entries, int G, int rank, int world,
                                                    const PeerTable& dst, const PeerTable& flags, unsigned long long epoch,
                                                    unsigned long long* status, long long* route_stats, int* hist) {
  if (threadIdx.x == 0) trace_mark(status, TR_LOADS);
  if (route_stats != nullptr && threadIdx.x < 4) route_stats[threadIdx.x] = 0;
  #pragma unroll 1
  for (int g = threadIdx.x; g < G; g += blockDim.x) hist[g] = 0;
  __syncthreads();
  #pragma unroll 1
  for (int n = threadIdx.x; n < n_entries; n += blockDim.x) {
    const int g = topk_own[n];
    if (g >= 0 && g < G) atomicAdd(&hist[g], 1);
    else if (g >= G && status) atomicOr(status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);   // negative: a pad copy
  }
  __syncthreads();
  #pragma unroll 1
  for (int p = 0; p < world; ++p) {
    int* row = reinterpret_cast<int*>(dst.ptr[p]) + (size_t)rank * G;
    #pragma unroll 1
    for (int g = threadIdx.x; g < G; g += blockDim.x) row[g] = hist[g];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world && flags.ptr[threadIdx.x] != nullptr)
    st_relaxed_sys(reinterpret_cast<unsigned long long*>(flags.ptr[threadIdx.x]) + rank, epoch);
}

__global__ void loads_publish_kernel(const int* __restrict__ topk_own, int n_entries, int G, int rank, int world,
                                     PeerTable dst0, PeerTable dst1, PeerTable flags, unsigned long long* ctr,
                                     unsigned long long* status, long long* route_stats) {
  extern __shared__ int hist[];
  const unsigned long long epoch = step_epoch(ctr, true);      // first kernel of a step
  loads_publish_block(topk_own, n_entries, G, rank, world, (epoch & 1) ? dst1 : dst0, flags, epoch, status, route_stats, hist);
  if (threadIdx.x == 0 && ctr != nullptr) *ctr = epoch;
}

// Thread 0 of a block waits until every rank's word in `flags` reached `epoch`.
__device__ __forceinline__ bool block_wait_all(const unsigned long long* flags, int world, unsigned long long epoch,
                                               unsigned long long limit_ns, unsigned long long* status, int what) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (flags != nullptr && threadIdx.x < world) {
    if (!wait_epoch_geq(flags + threadIdx.x, epoch, limit_ns)) {
      record_timeout(status, what, threadIdx.x, (long long)epoch);
      ok_s = 0;
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------
// route: one warp per expert.
//   lane 0   replica table (ascending host rank), bounds U / Lb, R-round rotation water-fill
//            (python/zepp/routing.py:80-119; device twin src/planner/routing.cu:75-234);
//   lanes    release / extra budgets of this source per replica by largest remainder
//            (routing.py:189-225);
//   warp     deterministic ordinal assignment of this source's entries (routing.py:146-186):
//            the o-th entry of expert g in flat (token, k) order goes to the visit-ordered
//            segment that contains o.  Ordinals come from ballots over the entry stream.
// ---------------------------------------------------------------------------------------
struct RouteArgs {
  const int* topk_own;      // [S*K]
  int n_entries;
  const int* loads;         // [R, G]
  const int* loads_odd;     // the odd-epoch copy of the table when `epoch_ptr` is set (else unused)
  const int* l2p;           // [G, R]
  const int* lcnts;         // [G]
  int G, R, L, nlp, my_rank;
  long long c_num, c_den;
  int* ws;
  int* phys_own;            // [S*K]
  const unsigned long long* loads_flags;   // [R] or nullptr
  const unsigned long long* epoch_ptr;     // device step counter or nullptr (stand-alone use)
  unsigned long long limit_ns;
  unsigned long long* status;
  long long* stats;         // [4]: 0 stranded rows, 1 vacate moves, 2 ordinal overflow, 3 unused
};

__global__ void __launch_bounds__(256) route_kernel(RouteArgs a) {
  const unsigned long long epoch = step_epoch(a.epoch_ptr, false);
  if (a.epoch_ptr != nullptr && (epoch & 1)) a.loads = a.loads_odd;
  if (!block_wait_all(a.loads_flags, a.R, epoch, a.limit_ns, a.status, WAIT_LOADS)) return;
  const int warps_per_block = blockDim.x >> 5;
  const int wib = threadIdx.x >> 5;
  const int g = blockIdx.x * warps_per_block + wib;
  const int lane = threadIdx.x & 31;
  const int R = a.R, L = a.L, NN = R / L, G = a.G;
  // ---- entries of single-replica experts need no ordinal: every thread of the grid fills a
  //      slice of them straight from the placement (the only replica is the first valid l2p entry)
  if (a.topk_own != nullptr)
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < a.n_entries; n += gridDim.x * blockDim.x) {
    const int e = a.topk_own[n];
    if (e < 0 || e >= G) { a.phys_own[n] = -1; continue; }     // pad copy (or an id the loads kernel reported)
    const int cnt = min(a.lcnts[e], R);
    int found = 0, p0 = -1;
    for (int j = 0; j < cnt; ++j) {
      const int p = a.l2p[e * R + j];
      if (p >= 0) { if (found == 0) p0 = p; ++found; }
    }
    if (found == 1) a.phys_own[n] = p0;
  }
  if (g >= a.G) return;
  const int CM = route_cm(R);
  const RouteWs w = route_ws_layout(G, R);
  int* rep = a.ws + w.rep + g * CM;
  int* rphys = a.ws + w.rphys + g * CM;
  int* fillp = a.ws + w.fill + g * CM;
  int* Mg = a.ws + w.M + (size_t)g * R * CM;
  int* relp = a.ws + w.rel + g * CM;
  int* extp = a.ws + w.ext + g * CM;
  __shared__ int left_s[8][kMaxRanks];
  __shared__ long long fill_s[8][kMaxRep];
  __shared__ int cum_s[8][kMaxRep];
  __shared__ int vphys_s[8][kMaxRep];
  int* left = left_s[wib];
  long long* fill = fill_s[wib];

  // ---- replica table + bounds + water-fill (lane 0)
  int c = 0;
  long long D = 0, U = 0, Lb = 0;
  if (lane == 0) {
    const int cnt = min(a.lcnts[g], R);
    for (int j = 0; j < cnt; ++j) {
      const int p = a.l2p[g * R + j];
      if (p >= 0 && c < CM) { rep[c] = p / a.nlp; rphys[c] = p; ++c; }
    }
    for (int j = c; j < CM; ++j) { rep[j] = -1; rphys[j] = -1; }
    for (int i = 0; i < R; ++i) { left[i] = a.loads[i * G + g]; D += left[i]; }
    if (c > 0) {
      U = ceil_div_ll((a.c_den + a.c_num) * D, a.c_den * c);
      Lb = ((a.c_den - a.c_num) * D) / (a.c_den * c);
    }
    for (int j = 0; j < CM; ++j) fill[j] = 0;
    for (int i = 0; i < R; ++i)
      for (int j = 0; j < CM; ++j) Mg[i * CM + j] = 0;
    long long unassigned = D;
    for (int p = 0; p < R && c > 0; ++p) {
      const int du = p / L, dl = p % L;
      for (int jj = 0; jj < c; ++jj) {
        const int j = rep[jj];
        const int i = ((((j / L) - du) % NN + NN) % NN) * L + ((((j % L) - dl) % L + L) % L);
        long long def_others = 0;
        for (int k = 0; k < c; ++k)
          if (k != jj && Lb > fill[k]) def_others += Lb - fill[k];
        long long take = left[i];
        if (U - fill[jj] < take) take = U - fill[jj];
        if (unassigned - def_others < take) take = unassigned - def_others;
        if (take < 0) take = 0;
        Mg[i * CM + jj] = (int)take;
        fill[jj] += take;
        left[i] -= (int)take;
        unassigned -= take;
      }
    }
    if (unassigned != 0) {
      if (a.stats) atomicAdd((unsigned long long*)a.stats + 0, (unsigned long long)unassigned);
      if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_ROUTE);
    }
    a.ws[w.c + g] = c;
    a.ws[w.D + g] = (int)D;
    a.ws[w.U + g] = (int)U;
    a.ws[w.Lb + g] = (int)Lb;
    for (int j = 0; j < CM; ++j) fillp[j] = (int)fill[j];
  }
  c = __shfl_sync(0xffffffffu, c, 0);
  U = __shfl_sync(0xffffffffu, U, 0);
  Lb = __shfl_sync(0xffffffffu, Lb, 0);
  __syncwarp();

  // ---- budgets of this source (lane jj)
  const int me = a.my_rank;
  if (lane < CM) {
    long long rel = 0, ext = 0;
    if (lane < c) {
      const long long f = fill[lane];
      if (f > Lb) {            // release: split fill - Lb by the takes M[g][.][jj]
        const long long total = f - Lb;
        long long Wsum = 0;
        for (int k = 0; k < R; ++k) Wsum += Mg[k * CM + lane];
        if (Wsum > 0) {
          const long long wi = Mg[me * CM + lane];
          long long base_sum = 0;
          int pos = 0;
          const long long fi = (total * wi) % Wsum;
          for (int k = 0; k < R; ++k) {
            const long long wk = Mg[k * CM + lane];
            base_sum += (total * wk) / Wsum;
            const long long fk = (total * wk) % Wsum;
            if (fk > fi || (fk == fi && k < me)) ++pos;
          }
          rel = (total * wi) / Wsum + (pos < total - base_sum ? 1 : 0);
          if (rel > wi) rel = wi;
        }
      }
      if (U > f && R > 1) {    // extra: split U - fill by the demands d[.][g]
        // (a single rank gets no extra budget: the reference's table pass consumes its demand
        //  tensor in place when R == 1, python/zepp/routing.py:94,115,222)
        const long long total = U - f;
        long long Wsum = 0;
        for (int k = 0; k < R; ++k) Wsum += a.loads[k * G + g];
        if (Wsum > 0) {
          const long long wi = a.loads[me * G + g];
          long long base_sum = 0;
          int pos = 0;
          const long long fi = (total * wi) % Wsum;
          for (int k = 0; k < R; ++k) {
            const long long wk = a.loads[k * G + g];
            base_sum += (total * wk) / Wsum;
            const long long fk = (total * wk) % Wsum;
            if (fk > fi || (fk == fi && k < me)) ++pos;
          }
          ext = (total * wi) / Wsum + (pos < total - base_sum ? 1 : 0);
        }
      }
    }
    relp[lane] = (int)rel;
    extp[lane] = (int)ext;
  }

  if (a.topk_own == nullptr) return;
  if (c <= 1) return;
  // ---- visit order of this source and cumulative takes
  {
    int pr = 1 << 30;
    if (lane < c) {
      const int j = rep[lane];
      pr = ((((j / L) - (me / L)) % NN + NN) % NN) * L + ((((j % L) - (me % L)) % L + L) % L);
    }
    int pos = 0;
    for (int k = 0; k < c; ++k) {
      const int prk = __shfl_sync(0xffffffffu, pr, k);
      if (lane < c && (prk < pr || (prk == pr && k < lane))) ++pos;
    }
    if (lane < c) {
      cum_s[wib][pos] = Mg[me * CM + lane];
      vphys_s[wib][pos] = rphys[lane];
    }
    __syncwarp();
    if (lane == 0) {
      int acc = 0;
      for (int k = 0; k < c; ++k) { acc += cum_s[wib][k]; cum_s[wib][k] = acc; }
    }
    __syncwarp();
  }
  // ---- ordinal assignment over the entry stream
  int base = 0;
  for (int n0 = 0; n0 < a.n_entries; n0 += 32) {
    const int n = n0 + lane;
    const bool mine = n < a.n_entries && a.topk_own[n] == g;
    const unsigned bal = __ballot_sync(0xffffffffu, mine);
    if (mine) {
      const int o = base + __popc(bal & ((1u << lane) - 1u));
      int seg = 0;
      for (int k = 0; k < c; ++k) seg += (cum_s[wib][k] <= o) ? 1 : 0;
      if (seg < c) {
        a.phys_own[n] = vphys_s[wib][seg];
      } else {
        a.phys_own[n] = c > 0 ? vphys_s[wib][c - 1] : 0;
        if (a.stats) atomicAdd((unsigned long long*)a.stats + 2, 1ull);
        if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_ROUTE);
      }
    }
    base += __popc(bal);
  }
}

// ---------------------------------------------------------------------------------------
// vacate + routing exchange.
// route_vacate_kernel: one warp runs the per-token vacate pass of this source in token order
// with the host reference's semantics (python/zepp/routing.py:242-297: least-touched remote node
// first, targets = home then the other touched nodes in first-touch order, all-or-nothing per
// node, budgets paid on both replicas); launched only when the topology has more than one node.
// route_finish_kernel: every block copies the send row [phys | weight bits]
// (python/zepp/planner.py:122) into each rank's gather table; the last block publishes the epoch.
// ---------------------------------------------------------------------------------------
struct FinishArgs {
  const int* topk_own;     // [S*K]
  int* phys_own;           // [S*K] in/out
  const float* probs_own;  // [S*K]
  int S, K, G, R, L, nlp, my_rank;
  int* ws;
  int* send_row;           // [2*S*K] local copy of the row (may be nullptr)
  PeerTable dst;           // rank p's gather table [R, 2*S*K]; nullptr entries skipped
  PeerTable dst_odd;       // the odd-epoch tables
  PeerTable flags;         // rank p's arrival words [R]
  int world;               // ranks to publish to (0: none)
  const unsigned long long* epoch_ptr;
  unsigned int* block_counter;   // self-resetting arrival counter of the grid (nullptr: launched as one block)
  unsigned long long* status;
  long long* stats;
};

__device__ void vacate_serial(const FinishArgs& a) {
  const int R = a.R, L = a.L, K = a.K, nlp = a.nlp, G = a.G;
  const int CM = route_cm(R);
  const RouteWs w = route_ws_layout(G, R);
  const int home = a.my_rank / L;
  int* rel = a.ws + w.rel;
  int* ext = a.ws + w.ext;
  const int* rep = a.ws + w.rep;
  const int* rphys = a.ws + w.rphys;
  const int* cc = a.ws + w.c;
  long long moves = 0;
  int node_of[64];
  int grp_node[64], grp_cnt[64];
  int plan_k[64], plan_jo[64], plan_jt[64];
  const int Kc = K < 64 ? K : 64;
  for (int s = 0; s < a.S; ++s) {
    int* ph = a.phys_own + s * K;
    const int* tk = a.topk_own + s * K;
    bool any_remote = false;
    for (int k = 0; k < Kc; ++k) {
      node_of[k] = ph[k] < 0 ? home : ph[k] / nlp / L;          // a pad copy is never remote
      any_remote |= node_of[k] != home;
    }
    if (!any_remote) continue;
    for (int guard = 0; guard < 4 * Kc + 4; ++guard) {
      // remote nodes in first-touch order with their entry counts
      int ng = 0;
      for (int k = 0; k < Kc; ++k) {
        if (node_of[k] == home) continue;
        int q = 0;
        while (q < ng && grp_node[q] != node_of[k]) ++q;
        if (q == ng) { grp_node[ng] = node_of[k]; grp_cnt[ng] = 0; ++ng; }
        ++grp_cnt[q];
      }
      if (ng == 0) break;
      bool moved = false;
      // candidates by (entry count, node id) ascending
      unsigned long long tried = 0;
      for (int round = 0; round < ng && !moved; ++round) {
        int best = -1;
        for (int q = 0; q < ng; ++q) {
          if (tried >> q & 1ull) continue;
          if (best < 0 || grp_cnt[q] < grp_cnt[best] || (grp_cnt[q] == grp_cnt[best] && grp_node[q] < grp_node[best]))
            best = q;
        }
        tried |= 1ull << best;
        const int n = grp_node[best];
        int np = 0;
        bool ok = true;
        for (int k = 0; k < Kc && ok; ++k) {
          if (node_of[k] != n) continue;
          const int g = tk[k];
          const int c = cc[g];
          int jo = -1;
          for (int jj = 0; jj < c; ++jj)
            if (rphys[g * CM + jj] == ph[k]) { jo = jj; break; }
          if (jo < 0 || rel[g * CM + jo] <= 0) { ok = false; break; }
          int jt = -1;
          // targets: home, then the other touched nodes in first-touch order
          for (int ti = -1; ti < ng && jt < 0; ++ti) {
            int m;
            if (ti < 0) m = home;
            else { if (ti == best) continue; m = grp_node[ti]; }
            for (int jj = 0; jj < c; ++jj)
              if (rep[g * CM + jj] / L == m && ext[g * CM + jj] > 0) { jt = jj; break; }
          }
          if (jt < 0) { ok = false; break; }
          plan_k[np] = k; plan_jo[np] = jo; plan_jt[np] = jt; ++np;
        }
        if (!ok) continue;
        for (int q = 0; q < np; ++q) {
          const int k = plan_k[q], g = tk[k];
          rel[g * CM + plan_jo[q]] -= 1;
          ext[g * CM + plan_jo[q]] += 1;
          ext[g * CM + plan_jt[q]] -= 1;
          rel[g * CM + plan_jt[q]] += 1;
          ph[k] = rphys[g * CM + plan_jt[q]];
          node_of[k] = rep[g * CM + plan_jt[q]] / L;
          ++moves;
        }
        moved = true;
      }
      if (!moved) break;
    }
  }
  if (a.stats) a.stats[1] = moves;
}

// The same pass run by a block of warps, a lane per entry of a token (K <= 32).  The budgets are shared state, so
// tokens take effect in token order; but a token that cannot vacate any node changes nothing.  The block therefore
// looks at kVacWarps consecutive tokens at once, one warp each, against the budgets as they stand; tokens before
// the first one that can move are finished, that one runs its whole pass (it alone writes), and the block goes on
// behind it.  Within a token the group counts, the candidate choice and every entry's plan are warp operations;
// the budget tables sit in shared memory when they fit (`staged`), the token rows are staged `chunk` tokens at a
// time.  Results equal vacate_serial's bit for bit: a token's plan reads the budgets before any of its entries is
// applied, and the applies are atomic adds, which commute.
constexpr int kVacWarps = 16;

struct VacateShape {
  int staged;      // 1: rel | ext | (rphys | rep << 24) | c tables live in dynamic shared memory
  int chunk;       // tokens staged per round
  size_t smem;     // dynamic shared memory bytes of the launch
};

inline VacateShape vacate_shape(int G, int R, int K, int nlp, bool tables_in_global = false) {
  VacateShape v{};
  const size_t limit = 44 * 1024;
  const size_t tables = ((size_t)3 * G * route_cm(R) + G) * sizeof(int);
  const size_t row = (size_t)2 * (K < 1 ? 1 : K) * sizeof(int);
  v.staged = (!tables_in_global && tables + 8 * row <= limit && (long long)R * nlp < (1ll << 24)) ? 1 : 0;
  const size_t left = limit - (v.staged ? tables : 0);
  size_t chunk = left / row;
  if (chunk > 256) chunk = 256;
  v.chunk = (int)chunk;
  v.smem = (v.staged ? tables : 0) + chunk * row;
  return v;
}

struct VacateTabs {
  int* rel;              // budgets (shared or global)
  int* ext;
  const int* pk;         // staged: rphys | rep << 24 (else nullptr)
  const int* rep;        // global tables
  const int* rphys;
  const int* cc;         // replicas per expert
  int CM, L, nlp, home, K;
};

// One token, one warp.  dry: return true as soon as some node could be vacated, change nothing.
// Otherwise run the token's whole pass, write its row back and return the number of entries moved.
__device__ int vacate_token(const VacateTabs& v, int* row_ph, const int* row_tk, int* grp_node, bool dry) {
  const int lane = threadIdx.x & 31;
  const int K = v.K, L = v.L, CM = v.CM, home = v.home;
  // budgets are read where the atomics that change them land (never from a stale L1 line of the global tables)
  auto budget = [](const int* p) { return *reinterpret_cast<const volatile int*>(p); };
  const bool active = lane < K;
  int ph = active ? row_ph[lane] : -1;
  const int g = active ? row_tk[lane] : -1;
  int node = ph < 0 ? home : ph / v.nlp / L;          // a pad copy is never remote
  if (__ballot_sync(0xffffffffu, node != home) == 0) return 0;
  int moves = 0;
  for (int guard = 0; guard < 4 * K + 4; ++guard) {
    const bool is_remote = node != home;
    if (__ballot_sync(0xffffffffu, is_remote) == 0) break;
    const unsigned peers = __match_any_sync(0xffffffffu, node);      // the entries served on my node
    const int cnt = __popc(peers);
    const bool leader = is_remote && (__ffs(peers) - 1) == lane;     // first touch of a remote node
    const unsigned leaders = __ballot_sync(0xffffffffu, leader);
    const int ng = __popc(leaders);
    __syncwarp();
    if (leader) grp_node[__popc(leaders & ((1u << lane) - 1u))] = node;
    __syncwarp();
    unsigned tried = 0;
    bool moved = false;
    for (int round = 0; round < ng && !moved; ++round) {
      // least-touched remote node first, ties by node id
      const unsigned key = (leader && !((tried >> lane) & 1u)) ? ((unsigned)cnt << 16 | (unsigned)node) : 0xffffffffu;
      const unsigned best_key = __reduce_min_sync(0xffffffffu, key);
      const int best_lane = __ffs(__ballot_sync(0xffffffffu, key == best_key)) - 1;
      tried |= 1u << best_lane;
      const int n = (int)(best_key & 0xffffu);
      const int best_q = __popc(leaders & ((1u << best_lane) - 1u));
      const bool in = is_remote && node == n;
      bool ok = true;
      int jo = -1, jt = -1;
      if (in) {
        const int c = v.cc[g];
        const int base = g * CM;
        for (int jj = 0; jj < c; ++jj) {
          const int rp = v.pk ? (v.pk[base + jj] & 0xffffff) : v.rphys[base + jj];
          if (rp == ph) { jo = jj; break; }
        }
        if (jo < 0 || budget(v.rel + base + jo) <= 0) ok = false;
        // targets: home, then the other touched nodes in first-touch order
        for (int ti = -1; ok && ti < ng && jt < 0; ++ti) {
          if (ti == best_q) continue;
          const int m = ti < 0 ? home : grp_node[ti];
          for (int jj = 0; jj < c; ++jj) {
            const int rr = v.pk ? (v.pk[base + jj] >> 24) : v.rep[base + jj];
            if (rr / L == m && budget(v.ext + base + jj) > 0) { jt = jj; break; }
          }
        }
        if (jt < 0) ok = false;
      }
      if (__any_sync(0xffffffffu, in && !ok)) continue;       // all or nothing per node
      if (dry) return 1;
      if (in) {
        const int base = g * CM;
        atomicSub(&v.rel[base + jo], 1);
        atomicAdd(&v.ext[base + jo], 1);
        atomicSub(&v.ext[base + jt], 1);
        atomicAdd(&v.rel[base + jt], 1);
        ph = v.pk ? (v.pk[base + jt] & 0xffffff) : v.rphys[base + jt];
        node = (v.pk ? (v.pk[base + jt] >> 24) : v.rep[base + jt]) / L;
      }
      moves += __popc(__ballot_sync(0xffffffffu, in));
      moved = true;
      __syncwarp();
    }
    if (!moved) break;
  }
  if (!dry && moves > 0 && active) row_ph[lane] = ph;
  return dry ? 0 : moves;
}

__global__ void __launch_bounds__(kVacWarps * 32) route_vacate_kernel(FinishArgs a, int staged, int chunk) {
  if (blockIdx.x != 0) return;
  const int R = a.R, L = a.L, K = a.K, nlp = a.nlp, G = a.G;
  if (K > 32) {                 // more entries per token than lanes
    if (threadIdx.x == 0) vacate_serial(a);
    return;
  }
  extern __shared__ int vac_sm[];
  __shared__ int grp_node_s[kVacWarps][32];
  __shared__ int can_move_s[kVacWarps];
  __shared__ int moves_s;
  const int CM = route_cm(R);
  const RouteWs w = route_ws_layout(G, R);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int GC = G * CM;
  VacateTabs v{};
  v.rel = a.ws + w.rel; v.ext = a.ws + w.ext; v.pk = nullptr;
  v.rep = a.ws + w.rep; v.rphys = a.ws + w.rphys; v.cc = a.ws + w.c;
  v.CM = CM; v.L = L; v.nlp = nlp; v.home = a.my_rank / L; v.K = K;
  int* tok = vac_sm;
  if (tid == 0) moves_s = 0;
  if (staged) {
    int* rel = vac_sm;
    int* ext = vac_sm + GC;
    int* pk = vac_sm + 2 * GC;
    int* cs = vac_sm + 3 * GC;
    tok = cs + G;
    for (int i = tid; i < GC; i += blockDim.x) {
      rel[i] = a.ws[w.rel + i];
      ext[i] = a.ws[w.ext + i];
      pk[i] = (v.rphys[i] & 0xffffff) | (v.rep[i] << 24);
    }
    for (int i = tid; i < G; i += blockDim.x) cs[i] = v.cc[i];
    v.rel = rel; v.ext = ext; v.pk = pk; v.cc = cs;
  }
  int* tok_ph = tok;
  int* tok_tk = tok + chunk * K;
  int moves = 0;
  for (int s0 = 0; s0 < a.S; s0 += chunk) {
    const int ns = min(chunk, a.S - s0);
    __syncthreads();
    for (int i = tid; i < ns * K; i += blockDim.x) {
      tok_ph[i] = a.phys_own[(size_t)s0 * K + i];
      tok_tk[i] = a.topk_own[(size_t)s0 * K + i];
    }
    __syncthreads();
    int t = 0;
    while (t < ns) {
      const int mine = t + warp;
      int can = 0;
      if (mine < ns) can = vacate_token(v, tok_ph + mine * K, tok_tk + mine * K, grp_node_s[warp], true);
      if (lane == 0) can_move_s[warp] = can;
      __syncthreads();
      int first = kVacWarps;
      for (int q = kVacWarps - 1; q >= 0; --q)
        if (can_move_s[q]) first = q;
      if (first < kVacWarps) {
        if (warp == first) moves += vacate_token(v, tok_ph + mine * K, tok_tk + mine * K, grp_node_s[warp], false);
        t += first + 1;
      } else {
        t += kVacWarps;
      }
      __syncthreads();
    }
    for (int i = tid; i < ns * K; i += blockDim.x) a.phys_own[(size_t)s0 * K + i] = tok_ph[i];
  }
  if (lane == 0 && moves) atomicAdd(&moves_s, moves);
  __syncthreads();
  if (staged)
    for (int i = tid; i < GC; i += blockDim.x) {
      a.ws[w.rel + i] = v.rel[i];
      a.ws[w.ext + i] = v.ext[i];
    }
  if (tid == 0 && a.stats) a.stats[1] = moves_s;
}

__global__ void route_finish_kernel(FinishArgs a) {
  const int SK = a.S * a.K;
  const unsigned long long epoch = step_epoch(a.epoch_ptr, false);
  const PeerTable& dst = (epoch & 1) ? a.dst_odd : a.dst;
  const int* wbits = reinterpret_cast<const int*>(a.probs_own);
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < 2 * SK; n += gridDim.x * blockDim.x) {
    const int v = n < SK ? a.phys_own[n] : wbits[n - SK];
    if (a.send_row) a.send_row[n] = v;
    for (int p = 0; p < a.world; ++p)
      if (dst.ptr[p]) reinterpret_cast<int*>(dst.ptr[p])[(size_t)a.my_rank * 2 * SK + n] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool last = a.block_counter == nullptr || atomicInc(a.block_counter, gridDim.x - 1) == gridDim.x - 1;
    if (last) {
      __threadfence_system();
      for (int p = 0; p < a.world; ++p)
        if (a.flags.ptr[p]) st_relaxed_sys(reinterpret_cast<unsigned long long*>(a.flags.ptr[p]) + a.my_rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Single-replica fast path: when no expert has more than one instance (every one-node
// topology: the placement caps replicas at one per node) the water-fill is the identity --
// every copy of expert g goes to its only slot -- and neither the tables nor the gathered loads
// have a consumer (unless the swap decision wants the loads).  One kernel: phys = first valid
// l2p entry of the copy's expert, send row [phys | weight bits] into every rank's gather table,
// epoch flag by the last block.  It is the first kernel of the step when the loads exchange is
// skipped (first = 1) and then commits the step counter.
// ---------------------------------------------------------------------------------------
struct SimpleRouteArgs {
  const int* topk_own;
  const float* probs_own;
  const int* slot_of;      // [G] the only physical slot of every expert (-1: none)
  int SK, G, R, my_rank, world, first;
  int* phys_own;
  int* send_row;
  PeerTable dst, dst_odd, flags;
  unsigned long long* ctr;
  unsigned int* block_counter;
  unsigned long long* status;
  // optional: publish this rank's x in the same launch (blocks route_blocks .. gridDim-1 copy it)
  int route_blocks;
  const uint4* x;
  uint4* xsym_even;
  uint4* xsym_odd;
  size_t x_vec;
  PeerTable x_flags;
};

__device__ __forceinline__ int single_replica_slot(const SimpleRouteArgs& a, const int* slots, int e) {
  if (e < 0) return -1;                    // pad copy: no slot, no owner
  if (e >= a.G) {
    if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_BAD_INDEX);
    return -1;
  }
  const int p = slots[e];
  if (p < 0) {
    if (a.status) atomicOr(a.status + ST_ERROR, (unsigned long long)ERR_ROUTE);
    return -1;
  }
  return p;
}

// slot_of[e] = first valid l2p entry of expert e (the placement's only replica when c_max == 1)
__global__ void slot_table_kernel(const int* l2p, const int* lcnts, int G, int R, int* slot_of) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= G) return;
  const int cnt = min(lcnts[e], R);
  int p0 = -1;
  for (int j = 0; j < cnt && p0 < 0; ++j)
    if (l2p[e * R + j] >= 0) p0 = l2p[e * R + j];
  slot_of[e] = p0;
}

// Rows [blk, nblk) of the single-replica routing: slot lookup, local copies, and the send row [phys | weight
// bits] into every rank's gather table.  `slots` is a shared-memory copy of slot_of.
__device__ void route_simple_rows(const SimpleRouteArgs& a, const int* slots, int blk, int nblk,
                                  unsigned long long epoch) {
  const PeerTable& dst = (epoch & 1) ? a.dst_odd : a.dst;
  const int* wbits = reinterpret_cast<const int*>(a.probs_own);
  const int SK = a.SK;
  const size_t row_off = (size_t)a.my_rank * 2 * SK;
  if ((SK & 3) == 0) {
    // four entries per thread, 16-byte stores into every rank's gather table
    #pragma unroll 1
    for (int q = blk * blockDim.x + threadIdx.x; q < SK / 4; q += nblk * blockDim.x) {
      const int4 e4 = reinterpret_cast<const int4*>(a.topk_own)[q];
      const int4 w4 = reinterpret_cast<const int4*>(wbits)[q];
      int4 p4;
      p4.x = single_replica_slot(a, slots, e4.x);
      p4.y = single_replica_slot(a, slots, e4.y);
      p4.z = single_replica_slot(a, slots, e4.z);
      p4.w = single_replica_slot(a, slots, e4.w);
      reinterpret_cast<int4*>(a.phys_own)[q] = p4;
      if (a.send_row) {
        reinterpret_cast<int4*>(a.send_row)[q] = p4;
        reinterpret_cast<int4*>(a.send_row + SK)[q] = w4;
      }
      #pragma unroll 1
      for (int p = 0; p < a.world; ++p) {
        int* row = reinterpret_cast<int*>(dst.ptr[p]) + row_off;
        reinterpret_cast<int4*>(row)[q] = p4;
        reinterpret_cast<int4*>(row + SK)[q] = w4;
      }
    }
  } else {
    #pragma unroll 1
    for (int n = blk * blockDim.x + threadIdx.x; n < SK; n += nblk * blockDim.x) {
      const int p0 = single_replica_slot(a, slots, a.topk_own[n]);
      const int wb = wbits[n];
      a.phys_own[n] = p0;
      if (a.send_row) { a.send_row[n] = p0; a.send_row[SK + n] = wb; }
      #pragma unroll 1
      for (int p = 0; p < a.world; ++p) {
        int* row = reinterpret_cast<int*>(dst.ptr[p]) + row_off;
        row[n] = p0;
        row[SK + n] = wb;
      }
    }
  }
}

__global__ void __launch_bounds__(256) route_simple_publish_kernel(SimpleRouteArgs a) {
  const unsigned long long epoch = step_epoch(a.ctr, a.first != 0);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    trace_mark(a.status, TR_ROUTE);
    trace_mark(a.status, TR_RING + (int)(epoch & 15));
  }
  extern __shared__ int slots[];             // [G] staged copy of the slot table (routing blocks)
  if ((int)blockIdx.x < a.route_blocks) {
    for (int g = threadIdx.x; g < a.G; g += blockDim.x) slots[g] = a.slot_of[g];
    __syncthreads();
    route_simple_rows(a, slots, blockIdx.x, a.route_blocks, epoch);
  } else {
    // x publication blocks
    uint4* xsym = (epoch & 1) ? a.xsym_odd : a.xsym_even;
    const size_t nb = gridDim.x - a.route_blocks;
    for (size_t i = (size_t)(blockIdx.x - a.route_blocks) * blockDim.x + threadIdx.x; i < a.x_vec; i += nb * blockDim.x)
      xsym[i] = a.x[i];
  }
  // one fence per block (thread 0, after the block barrier) orders every thread's stores before the
  // block's arrival; the last block to arrive publishes the epoch words
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicInc(a.block_counter, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) {
        st_relaxed_sys(reinterpret_cast<unsigned long long*>(a.flags.ptr[p]) + a.my_rank, epoch);
        if (a.x != nullptr) st_relaxed_sys(reinterpret_cast<unsigned long long*>(a.x_flags.ptr[p]) + a.my_rank, epoch);
      }
      if (a.first && a.ctr != nullptr) *a.ctr = epoch;
    }
  }
}

}  // namespace zepp
