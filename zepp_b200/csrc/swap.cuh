// Band-triggered intra-node expert swap: decision and swap-lane metadata, single launches.
// The decision restates python/zepp/swap.py:36-201 (decide_swaps with one exchange per pair and
// round, net_moves, rebuild_l2p) on the device, as src/planner/swap_decide.cu:81-346 does; the
// result block keeps that kernel's layout.  lane_arm follows src/planner/lane_device.cu:49-80 as
// pinned by tests/test_lane_device.py:36-58.
#pragma once
#include "common.cuh"
#include "planner.cuh"

namespace zepp {

constexpr int kSwapThreads = 256;
constexpr int kSwapMaxL = 16;
constexpr long long kSwapBig = 1ll << 60;

struct SwapArgs {
  const int* loads;     // [R, G]
  int* p2l;             // [R*nlp] in/out
  int* l2p;             // [G, R] in/out
  const int* lcnts;     // [G]
  int R, G, L, nlp, cap, max_rounds;
  double C;
  long long* out;       // [3 + R + 4*R*cap + R*nlp + G]
  // ---- inside a layer step (all nullptr / 0 for the stand-alone entry point)
  const int* loads_odd;                    // the loads table of odd epochs (picked on the device, like the router does)
  const unsigned long long* epoch_ptr;     // device step counter
  const unsigned long long* loads_flags;   // [R] arrival words of the loads exchange (waited for here), or nullptr
  unsigned long long limit_ns;
  unsigned long long* status;
  int* slot_of;         // [G] out: the first valid l2p entry of every expert on the placement this step routes on
  int rank;
  int* sched;           // [gpe] out: schedule word per local group (bit 30 = slot received an expert this step)
  int first;            // the calling kernel is the step's first: the epoch is *epoch_ptr + 1 (not committed yet)
  int* redirect;        // [gpe] out: group whose weights the GEMMs read: the group itself, or gpe + i for the i-th incoming expert
  unsigned int* ready;  // [2 * cap] out: zeroed chunk counters of the staging entries (W1, then W2)
};

__device__ __forceinline__ bool band_out(const long long* Lr, int n, int L, double C) {
  long long tot = 0, mx = -kSwapBig;
  for (int j = 0; j < L; ++j) {
    const long long v = Lr[n * L + j];
    tot += v;
    if (v > mx) mx = v;
  }
  return (double)mx * (double)L > (1.0 + C) * (double)tot;
}

__device__ __forceinline__ void slot_key(const int* cur, const long long* w, int s, bool heavy, long long& k1,
                                         long long& k2) {
  const int e = cur[s];
  if (e >= 0) { k1 = heavy ? -w[s] : w[s]; k2 = e; }
  else { k1 = kSwapBig; k2 = kSwapBig; }
}

// Tables the rest of a layer step reads, from the placement `cur` the decision left ([R*nlp] experts per slot):
// slot_of (the router's slot lookup) and, for this rank, which groups received an expert (their tiles are
// scheduled last and read their weights from the staging entries until the step's end).
__device__ void swap_step_tables(const SwapArgs& a, const int* cur, int cnt, const long long* mv) {
  const int NS = a.R * a.nlp, gpe = a.nlp + 1;
  if (a.slot_of != nullptr) {
    #pragma unroll 1
    for (int e = threadIdx.x; e < a.G; e += blockDim.x) {
      int p0 = -1;
      #pragma unroll 1
      for (int s = 0; s < NS && p0 < 0; ++s)
        if (cur[s] == e) p0 = s;
      a.slot_of[e] = p0;
    }
  }
  if (threadIdx.x == 0 && a.epoch_ptr != nullptr) trace_mark(a.status, TR_DECIDE_END);
  if (a.ready != nullptr)
    #pragma unroll 1
    for (int i = threadIdx.x; i < 2 * a.cap; i += blockDim.x) a.ready[i] = 0u;
  if (a.sched != nullptr) {
    #pragma unroll 1
    for (int g = threadIdx.x; g < gpe; g += blockDim.x) {
      int hit = -1;
      #pragma unroll 1
      for (int i = 0; i < cnt; ++i)
        if ((int)mv[4 * i] == g - 1) hit = i;
      a.sched[g] = hit >= 0 ? (1 << 30) : 0;
      a.redirect[g] = hit >= 0 ? gpe + hit : g;
    }
  }
}

// The decision by one block of any size (shared memory: swap_decide_smem_bytes for that size).
__device__ void swap_decide_body(SwapArgs a, long long* sm64) {
  const int R = a.R, G = a.G, L = a.L, nlp = a.nlp, NS = R * nlp, NN = R / L, P = L / 2, Q = NN * P;
  long long* lg = sm64;                 // [G]
  long long* w = lg + G;                // [NS]
  long long* Lr = w + NS;               // [R]
  int* a0 = (int*)(Lr + R);             // [NS]
  int* cur = a0 + NS;                   // [NS]
  int* Hh = cur + NS;                   // [Q]
  int* Lo = Hh + (Q > 0 ? Q : 1);       // [Q]
  int* sw = Lo + (Q > 0 ? Q : 1);       // [Q][5]: has, slot_h, e_h, slot_l, e_l
  int* node_out = sw + 5 * (Q > 0 ? Q : 1);   // [NN]
  int* cand = node_out + NN;            // [warps][2][8]
  __shared__ int s_any, s_stop, s_rounds;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, wid = tid >> 5, nw = nt >> 5;
  const int off_cnt = 3, off_mv = 3 + R, off_p2l = off_mv + 4 * R * a.cap, off_lg = off_p2l + NS;
  if (a.epoch_ptr != nullptr) {
    const unsigned long long epoch = step_epoch(a.epoch_ptr, a.first != 0);
    if (epoch & 1) a.loads = a.loads_odd;
    if (tid == 0) trace_mark(a.status, TR_DECIDE);
    if (!block_wait_all(a.loads_flags, R, epoch, a.limit_ns, a.status, WAIT_LOADS)) return;
    if (tid == 0) trace_mark(a.status, TR_DECIDE_GO);
  }

  #pragma unroll 1
  for (int e = tid; e < G; e += nt) {
    long long s = 0;
    #pragma unroll 4
    for (int r = 0; r < R; ++r) s += a.loads[r * G + e];
    lg[e] = s;
  }
  #pragma unroll 1
  for (int s = tid; s < NS; s += nt) { a0[s] = a.p2l[s]; cur[s] = a0[s]; }
  __syncthreads();
  #pragma unroll 1
  for (int s = tid; s < NS; s += nt) {
    const int e = a0[s];
    long long lc = e >= 0 ? a.lcnts[e] : 1;
    if (lc < 1) lc = 1;
    w[s] = e >= 0 ? lg[e] / lc : 0;
  }
  __syncthreads();
  #pragma unroll 1
  for (int r = tid; r < R; r += nt) {
    long long s = 0;
    #pragma unroll 1
    for (int j = 0; j < nlp; ++j) s += w[r * nlp + j];
    Lr[r] = s;
  }
  if (tid == 0) { s_any = 0; s_stop = 0; s_rounds = 0; }
  __syncthreads();
  #pragma unroll 1
  for (int n = tid; n < NN; n += nt) {
    node_out[n] = band_out(Lr, n, L, a.C) ? 1 : 0;
    if (node_out[n]) atomicOr(&s_any, 1);
  }
  __syncthreads();
  #pragma unroll 1
  for (int e = tid; e < G; e += nt) a.out[off_lg + e] = lg[e];

  if (s_any && Q > 0 && L <= kSwapMaxL) {
    #pragma unroll 1
    for (int round = 0; round < a.max_rounds; ++round) {
      // pairs: k-th heaviest with k-th lightest rank of every node (stable by key -Lr*L + l)
      #pragma unroll 1
      for (int n = tid; n < NN; n += nt) {
        int ord[kSwapMaxL];
        #pragma unroll 1
        for (int l = 0; l < L; ++l) ord[l] = l;
        #pragma unroll 1
        for (int i = 1; i < L; ++i) {
          const int v = ord[i];
          const long long kv = -Lr[n * L + v] * L + v;
          int j = i - 1;
          while (j >= 0 && (-Lr[n * L + ord[j]] * L + ord[j]) > kv) { ord[j + 1] = ord[j]; --j; }
          ord[j + 1] = v;
        }
        #pragma unroll 1
        for (int q = 0; q < P; ++q) { Hh[n * P + q] = n * L + ord[q]; Lo[n * P + q] = n * L + ord[L - 1 - q]; }
      }
      __syncthreads();
      #pragma unroll 1
      for (int q = wid; q < Q; q += nw) {
        const int h = Hh[q], lo = Lo[q];
        const long long LH = Lr[h], LL = Lr[lo];
        int* ch = cand + wid * 16;
        int* cl = ch + 8;
        const int Kc = nlp < 8 ? nlp : 8;
        bool pair_ok = (LH - LL > 1) && node_out[h / L];
        if (pair_ok) {
          #pragma unroll 1
          for (int side = 0; side < 2; ++side) {
            const int base = (side == 0 ? h : lo) * nlp;
            #pragma unroll 1
            for (int t = lane; t < nlp; t += 32) {
              long long k1, k2;
              slot_key(cur, w, base + t, side == 0, k1, k2);
              int rank = 0;
              #pragma unroll 1
              for (int u = 0; u < nlp; ++u) {
                long long u1, u2;
                slot_key(cur, w, base + u, side == 0, u1, u2);
                if (u1 < k1 || (u1 == k1 && (u2 < k2 || (u2 == k2 && u < t)))) ++rank;
              }
              if (rank < Kc) (side == 0 ? ch : cl)[rank] = base + t;
            }
          }
        }
        __syncwarp();
        long long best = -kSwapBig;
        int best_idx = -1;
        if (pair_ok) {
          #pragma unroll 1
          for (int idx = lane; idx < Kc * Kc; idx += 32) {
            const int sh = ch[idx / Kc], sl = cl[idx % Kc];
            const int eh = cur[sh], el = cur[sl];
            const long long wh = w[sh], wl = w[sl];
            bool ok = eh >= 0 && el >= 0 && eh != el && wh > wl;
            if (ok) {
              #pragma unroll 1
              for (int u = 0; u < nlp; ++u)
                if (cur[lo * nlp + u] == eh || cur[h * nlp + u] == el) { ok = false; break; }
            }
            if (ok) {
              const long long n1 = LH - wh + wl, n2 = LL - wl + wh;
              const long long gain = (LH > LL ? LH : LL) - (n1 > n2 ? n1 : n2);
              if (gain >= 1) {
                const long long key = gain * ((long long)G * G + 1) - ((long long)eh * G + el);
                if (key > best) { best = key; best_idx = idx; }
              }
            }
          }
        }
        #pragma unroll 1
        for (int o = 16; o > 0; o >>= 1) {
          const long long ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
          if (ob > best || (ob == best && oi >= 0 && (best_idx < 0 || oi < best_idx))) { best = ob; best_idx = oi; }
        }
        if (lane == 0) {
          int* s5 = sw + 5 * q;
          s5[0] = best_idx >= 0 ? 1 : 0;
          if (best_idx >= 0) {
            const int sh = ch[best_idx / Kc], sl = cl[best_idx % Kc];
            s5[1] = sh; s5[2] = cur[sh]; s5[3] = sl; s5[4] = cur[sl];
          }
        }
        __syncwarp();
      }
      __syncthreads();
      if (tid == 0) {
        int n_sw = 0;
        #pragma unroll 1
        for (int q = 0; q < Q; ++q) n_sw += sw[5 * q];
        if (n_sw == 0) {
          s_stop = 1;
        } else {
          // changed slots per rank against the step's original placement, with the round applied
          bool over = false;
          #pragma unroll 1
          for (int r = 0; r < R && !over; ++r) {
            int changed = 0;
            #pragma unroll 1
            for (int j = 0; j < nlp; ++j) {
              const int s = r * nlp + j;
              int v = cur[s];
              #pragma unroll 1
              for (int q = 0; q < Q; ++q) {
                if (!sw[5 * q]) continue;
                if (sw[5 * q + 1] == s) v = sw[5 * q + 4];
                if (sw[5 * q + 3] == s) v = sw[5 * q + 2];
              }
              if (v != a0[s]) ++changed;
            }
            if (changed > a.cap) over = true;
          }
          if (over) {
            s_stop = 1;
          } else {
            #pragma unroll 1
            for (int q = 0; q < Q; ++q) {
              if (!sw[5 * q]) continue;
              cur[sw[5 * q + 1]] = sw[5 * q + 4];
              cur[sw[5 * q + 3]] = sw[5 * q + 2];
            }
            s_rounds += 1;
            #pragma unroll 1
            for (int q = 0; q < Q; ++q) {
              if (!sw[5 * q]) continue;
              #pragma unroll 1
              for (int z = 0; z < 2; ++z) {
                const int sx = sw[5 * q + (z == 0 ? 1 : 3)];
                const int e = cur[sx];
                long long lc = e >= 0 ? a.lcnts[e] : 1;
                if (lc < 1) lc = 1;
                const long long wn = e >= 0 ? lg[e] / lc : 0;
                Lr[sx / nlp] += wn - w[sx];
                w[sx] = wn;
              }
            }
            #pragma unroll 1
            for (int n = 0; n < NN; ++n) node_out[n] = band_out(Lr, n, L, a.C) ? 1 : 0;
          }
        }
      }
      __syncthreads();
      if (s_stop) break;
    }
  }
  __syncthreads();
  const int rounds = s_rounds;
  if (rounds == 0) {
    if (tid == 0) { a.out[0] = 0; a.out[1] = 0; a.out[2] = 0; }
    #pragma unroll 1
    for (int r = tid; r < R; r += nt) a.out[off_cnt + r] = 0;
    #pragma unroll 1
    for (int s = tid; s < NS; s += nt) a.out[off_p2l + s] = a0[s];
    swap_step_tables(a, cur, 0, nullptr);
    return;
  }
  #pragma unroll 1
  for (int s = tid; s < NS; s += nt) { a.out[off_p2l + s] = cur[s]; a.p2l[s] = cur[s]; }
  #pragma unroll 1
  for (int e = tid; e < G; e += nt) {          // l2p: slots of every expert, ascending
    int j = 0;
    #pragma unroll 1
    for (int s = 0; s < NS; ++s)
      if (cur[s] == e && j < R) a.l2p[e * R + j++] = s;
    #pragma unroll 1
    for (; j < R; ++j) a.l2p[e * R + j] = -1;
  }
  __shared__ int s_total, s_err;
  if (tid == 0) { s_total = 0; s_err = 0; }
  __syncthreads();
  #pragma unroll 1
  for (int r = tid; r < R; r += nt) {          // pull lists, sorted by destination slot
    int cnt = 0;
    const int node = r / L;
    #pragma unroll 1
    for (int j = 0; j < nlp; ++j) {
      const int e = cur[r * nlp + j];
      if (e < 0 || a0[r * nlp + j] == e) continue;
      int sr = -1, ss = -1;
      #pragma unroll 1
      for (int s = node * L * nlp; s < (node + 1) * L * nlp; ++s)
        if (a0[s] == e) { sr = s / nlp; ss = s % nlp; }
      if (cnt < a.cap && sr >= 0) {
        long long* mv = a.out + off_mv + ((size_t)r * a.cap + cnt) * 4;
        mv[0] = j; mv[1] = sr; mv[2] = ss; mv[3] = e;
        ++cnt;
      } else {
        atomicOr(&s_err, 1);
      }
    }
    a.out[off_cnt + r] = cnt;
    atomicAdd(&s_total, cnt);
  }
  __syncthreads();
  if (tid == 0) { a.out[0] = rounds; a.out[1] = s_total; a.out[2] = s_err; }
  if (a.slot_of != nullptr || a.sched != nullptr) {
    __threadfence_block();
    __syncthreads();
    const int cnt = a.sched != nullptr ? min((int)a.out[off_cnt + a.rank], a.cap) : 0;
    swap_step_tables(a, cur, cnt, a.out + off_mv + (size_t)a.rank * a.cap * 4);
  }
}

__global__ void __launch_bounds__(kSwapThreads) swap_decide_kernel(SwapArgs a) {
  extern __shared__ long long swap_sm64[];
  swap_decide_body(a, swap_sm64);
}

__host__ __device__ inline size_t swap_decide_smem_bytes(int R, int G, int L, int nlp, int threads) {
  const int NS = R * nlp, NN = R / L, Q = NN * (L / 2) > 0 ? NN * (L / 2) : 1;
  return (size_t)(G + NS + R) * 8 + (size_t)(2 * NS + 7 * Q + NN + (threads / 32) * 16 + 8) * 4;
}

// Swap-lane metadata of one rank from the decision's result block: gate words of the unchanged
// slots (both weight matrices), the moved-last schedule word per group (bit 30 marks an incoming
// slot, the low bits rank the group inside its class; the pad group 0 counts as unchanged) and the
// staging addresses the GEMMs read incoming slots from.  A rank without incoming slots is untouched.
__global__ void lane_arm_kernel(const long long* out, int R, int rank, int nlp, int cap, long long* gate,
                                int* sched, long long* ovr0, long long* ovr1, const long long* stag,
                                long long epoch, const unsigned long long* epoch_ptr) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (epoch_ptr != nullptr) epoch = (long long)*epoch_ptr;      // the layer's device-resident step counter
  const int gpe = nlp + 1;
  const long long rounds = out[0];
  const int cnt = (int)out[3 + rank];
  if (rounds == 0 || cnt == 0) return;
  const long long* mv = out + 3 + R + (size_t)rank * cap * 4;
  for (int i = 0; i < cnt; ++i) {
    const int dj = (int)mv[4 * i];
    ovr0[1 + dj] = stag[i];
    ovr1[1 + dj] = stag[cap + i];
  }
  int f = 0, d = 0;
  for (int s = 0; s < gpe; ++s) {
    bool changed = false;
    if (s >= 1)
      for (int i = 0; i < cnt; ++i) changed |= (int)mv[4 * i] == s - 1;
    if (changed) {
      sched[s] = (1 << 30) | d;
      ++d;
    } else {
      sched[s] = f;
      ++f;
      if (s >= 1) { gate[s] = epoch; gate[gpe + s] = epoch; }
    }
  }
}


// ---------------------------------------------------------------------------------------
// Weight movement of a decided swap (replaces the copies of python/zepp/swap.py:508-559 and
// src/planner/lane_device.cu:82-163).  Nothing runs ahead of the step for it: the two GEMM kernels pull the
// incoming experts' W1 / W2 from the source ranks' slots into local staging groups with their spare warps while
// the other groups compute (csrc/gemm.cuh), the step's moved-in groups are scheduled last and read from staging,
// and the step's last kernel -- which starts its work only after every rank's combine GEMM has finished, so no
// rank still reads a slot -- copies staging into the destination slots (swap_commit below).  All of it is driven by
// the decision's result block on the device; a step without moves copies nothing.
// ---------------------------------------------------------------------------------------
struct SwapCommitArgs {
  const long long* block;                    // swap decision result block (nullptr: no swap in this layer)
  int R, rank, cap, gpe;
  size_t w1_vec, w2_vec;                     // 16-byte vectors per group of W1 / W2
  uint4* w1;                                 // [gpe + cap][w1_vec]: slot groups (group 0 = pad), then staging entries
  uint4* w2;
};

// staging -> destination slots, by every thread of the calling grid
__device__ __forceinline__ void swap_commit(const SwapCommitArgs& a) {
  if (a.block == nullptr) return;
  const long long rounds = a.block[0];
  int cnt = rounds > 0 ? (int)a.block[3 + a.rank] : 0;
  if (cnt > a.cap) cnt = a.cap;
  if (cnt <= 0) return;
  const long long* mv = a.block + 3 + a.R + (size_t)a.rank * a.cap * 4;
  const size_t per = a.w1_vec + a.w2_vec;
  const size_t total = (size_t)cnt * per;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / per);
    const size_t o = i - (size_t)m * per;
    const int dst = (int)mv[4 * m];
    if (o < a.w1_vec) a.w1[(size_t)(1 + dst) * a.w1_vec + o] = a.w1[(size_t)(a.gpe + m) * a.w1_vec + o];
    else a.w2[(size_t)(1 + dst) * a.w2_vec + (o - a.w1_vec)] = a.w2[(size_t)(a.gpe + m) * a.w2_vec + (o - a.w1_vec)];
  }
}

}  // namespace zepp
