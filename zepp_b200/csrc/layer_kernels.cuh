// Data-movement kernels around the two GEMMs: publication of x, the unfused dispatch pull and
// combine push of the `direct` strategy (comparison point; the reference's is
// python/zepp/comm/direct.py:184-213 over src/direct/all2all_single_2d_impl.cu), and the
// per-token top-k reduction (src/combine/combine_kernels.cu:440-478).
#pragma once
#include "common.cuh"
#include "planner.cuh"
#include "swap.cuh"

namespace zepp {

// x [S, H] -> this rank's symmetric buffer, then `epoch` into every rank's x_flags[rank].
__global__ void publish_x_kernel(const uint4* __restrict__ x, uint4* __restrict__ xsym_even,
                                 uint4* __restrict__ xsym_odd, size_t n_vec, int rank, int world, PeerTable flags,
                                 const unsigned long long* epoch_ptr, unsigned int* counter) {
  const unsigned long long epoch = step_epoch(epoch_ptr, false);
  uint4* xsym = (epoch & 1) ? xsym_odd : xsym_even;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x)
    xsym[i] = x[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicInc(counter, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        st_relaxed_sys(reinterpret_cast<unsigned long long*>(flags.ptr[p]) + rank, epoch);
    }
  }
}

// Staged dispatch push (overlap strategy, more than one rank).  As soon as a rank knows the owners
// of its own copies -- before the routing exchange -- it stores every token row once into the
// staging region stage[me] of each rank that owns at least one of the token's copies, at slot =
// number of earlier tokens of this rank that also go to that rank (the reference's pack-push dedup,
// src/dwire/dispatch_wire.cu:107-210 with the unique counts of python/zepp/routing.py:326-328).
// The NVLink transfer runs while the planning kernels run; the receiver derives the same slots from
// the gathered routing and its dispatch GEMM gathers from local memory.  Posted stores, no loads
// across NVLink.  A block owns a range of tokens; it recounts the slots of the tokens before its
// range from phys_own (a few KB) instead of waiting for another block.
struct PushArgs {
  const int* phys_own;                 // [S, K] physical slots of this rank's copies, or nullptr:
  const int* topk_own;                 //   then [S, K] expert ids looked up in slot_of (single-replica placements)
  const int* slot_of;                  // [G]
  int G;
  const __nv_bfloat16* x;              // [S, H]
  PeerTable stage;                     // rank p's staging buffer base [W, region_tokens, H]
  PeerTable flags;                     // rank p's push-arrival words [W]
  int S, K, H, nlp, rank, world;
  int region_tokens;                   // rows of one source's staging region (the layer's largest bucket)
  const unsigned long long* epoch_ptr;
  unsigned int* counter;
  unsigned long long* status;
};

constexpr int kPushMaxTokensPerBlock = 256;

// One block's share of the push: tokens [blk * tpb, (blk + 1) * tpb) of `nblk` equal ranges.  `epoch` is the
// step's epoch; the last of the nblk blocks to finish raises this rank's push flag on every rank.
__device__ void push_block(const PushArgs& a, int blk, int nblk, unsigned long long epoch) {
  __shared__ int before[kMaxRanks];      // tokens before this block's range that go to rank d
  __shared__ unsigned long long tmask[kPushMaxTokensPerBlock];
  __shared__ unsigned int dbits[kMaxRanks][kPushMaxTokensPerBlock / 32];   // bit t of row d: token t of the range goes to rank d
  __shared__ int wpre[kMaxRanks][kPushMaxTokensPerBlock / 32];             // such tokens in the earlier 32-token words
  const int tpb = (a.S + nblk - 1) / nblk;                    // tokens per block (<= kPushMaxTokensPerBlock)
  const int t_lo = min(a.S, blk * tpb);
  const int t_hi = min(a.S, t_lo + tpb);
  #pragma unroll 1
  for (int d = threadIdx.x; d < a.world; d += blockDim.x) before[d] = 0;
  __syncthreads();
  // owner masks of all tokens below t_hi: count those before the range, keep those inside it
  #pragma unroll 1
  for (int t = threadIdx.x; t < t_hi; t += blockDim.x) {
    unsigned long long m = 0;
    #pragma unroll 8
    for (int k = 0; k < a.K; ++k) {
      int p;
      if (a.phys_own != nullptr) {
        p = a.phys_own[t * a.K + k];
      } else {
        const int e = a.topk_own[t * a.K + k];
        p = (e >= 0 && e < a.G) ? a.slot_of[e] : -1;
      }
      if (p >= 0) m |= 1ull << (p / a.nlp);
    }
    if (t < t_lo) {
      while (m) { const int d = __ffsll((long long)m) - 1; m &= m - 1; atomicAdd(&before[d], 1); }
    } else {
      tmask[t - t_lo] = m;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int n_tok = t_hi - t_lo, n_words = (n_tok + 31) / 32;
  #pragma unroll 1
  for (int w = wid; w < n_words; w += nw) {
    const unsigned long long m = 32 * w + lane < n_tok ? tmask[32 * w + lane] : 0ull;
    #pragma unroll 1
    for (int d = 0; d < a.world; ++d) {
      const unsigned int bits = __ballot_sync(0xffffffffu, (m >> d) & 1ull);
      if (lane == 0) dbits[d][w] = bits;
    }
  }
  __syncthreads();
  #pragma unroll 1
  for (int d = threadIdx.x; d < a.world; d += blockDim.x) {
    int run = before[d];
    #pragma unroll 1
    for (int w = 0; w < n_words; ++w) { wpre[d][w] = run; run += __popc(dbits[d][w]); }
  }
  __syncthreads();
  // one warp per (token, destination) row
  const int vec_per_row = a.H / 8;
  const size_t region = (size_t)a.rank * a.region_tokens * a.H;
  #pragma unroll 1
  for (int pair = wid; pair < (t_hi - t_lo) * a.world; pair += nw) {
    const int tl = pair / a.world, d = pair - tl * a.world;
    const unsigned long long m = tmask[tl];
    if (!((m >> d) & 1ull)) continue;
    const int slot = wpre[d][tl >> 5] + __popc(dbits[d][tl >> 5] & ((1u << (tl & 31)) - 1u));
    const uint4* sp = reinterpret_cast<const uint4*>(a.x + (size_t)(t_lo + tl) * a.H);
    uint4* dp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.stage.ptr[d]) + region + (size_t)slot * a.H);
    #pragma unroll 1
    for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
      uint4 buf[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = v0 + q * 32 + lane;
        if (v < vec_per_row) buf[q] = sp[v];
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = v0 + q * 32 + lane;
        if (v < vec_per_row) dp[v] = buf[q];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicInc(a.counter, nblk - 1);
    if (prev == (unsigned int)nblk - 1) {
      __threadfence_system();
      #pragma unroll 1
      for (int p = 0; p < a.world; ++p)
        st_relaxed_sys(reinterpret_cast<unsigned long long*>(a.flags.ptr[p]) + a.rank, epoch);
    }
  }
}

__global__ void __launch_bounds__(256) dispatch_push_kernel(PushArgs a) {
  push_block(a, blockIdx.x, gridDim.x, step_epoch(a.epoch_ptr, false));
}

struct MoveArgs {
  const int* m_this;                       // [2] rows, first global row
  const int* row_tok;                      // [cap]
  const long long* row_dst;                // [cap]
  const __nv_bfloat16* const* x_ptrs;      // [W] symmetric x buffers (even epochs)
  const __nv_bfloat16* const* x_ptrs_odd;  // (odd epochs)
  const __nv_bfloat16* x_self;             // this rank's x (read directly)
  __nv_bfloat16* recv;                     // [cap, H]
  const __nv_bfloat16* staging;            // [cap, H]
  __nv_bfloat16* const* panels;            // [W]
  unsigned long long* const* done_flags;   // [W]
  const unsigned long long* x_flags;       // [W]
  unsigned int* counter;
  int H, S, world, rank, recv_cap;
  const unsigned long long* epoch_ptr;
  unsigned long long limit_ns;
  unsigned long long* status;
};

__device__ __forceinline__ void copy_row_warp(const uint4* sp, uint4* dp, int vec_per_row, int lane) {
  for (int v0 = 0; v0 < vec_per_row; v0 += 32 * 8) {
    uint4 buf[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int v = v0 + q * 32 + lane;
      if (v < vec_per_row) buf[q] = sp[v];
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int v = v0 + q * 32 + lane;
      if (v < vec_per_row) dp[v] = buf[q];
    }
  }
}

// recv[r] = x of row r's source token, pulled over NVLink (one warp per row).
__global__ void dispatch_pull_kernel(MoveArgs a) {
  const unsigned long long epoch = step_epoch(a.epoch_ptr, false);
  if (!block_wait_all(a.x_flags, a.world, epoch, a.limit_ns, a.status, WAIT_X)) return;
  if (a.status[ST_VIOLATION] != 0ull) return;
  const int m = min(a.m_this[0], a.recv_cap);
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < m; r += gridDim.x * wpb) {
    const int tok = a.row_tok[r];
    const int src = tok / a.S;
    const int t = tok - src * a.S;
    if (tok < 0 || src >= a.world) continue;
    const __nv_bfloat16* base = (src == a.rank && a.x_self != nullptr)
                                    ? a.x_self : ((epoch & 1) ? a.x_ptrs_odd[src] : a.x_ptrs[src]);
    copy_row_warp(reinterpret_cast<const uint4*>(base + (size_t)t * a.H),
                  reinterpret_cast<uint4*>(a.recv + (size_t)r * a.H), a.H / 8, lane);
  }
}

// staging[r] -> the home rank's slot panel, then the completion epoch to every rank.
__global__ void combine_push_kernel(MoveArgs a) {
  const unsigned long long epoch = step_epoch(a.epoch_ptr, false);
  const int m = a.status[ST_VIOLATION] != 0ull ? 0 : min(a.m_this[0], a.recv_cap);
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < m; r += gridDim.x * wpb) {
    const long long dst = a.row_dst[r];
    const int home = (int)(dst >> 40);
    if (dst < 0 || home >= a.world) continue;
    copy_row_warp(reinterpret_cast<const uint4*>(a.staging + (size_t)r * a.H),
                  reinterpret_cast<uint4*>(a.panels[home] + (size_t)(dst & ((1ll << 40) - 1))), a.H / 8, lane);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicInc(a.counter, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_relaxed_sys(a.done_flags[p] + a.rank, epoch);
    }
  }
}

// y[t] = bf16( sum_k float(panel[t, k]) ), once every rank's combine rows have landed.
__global__ void combine_reduce_kernel(const __nv_bfloat16* __restrict__ panel, __nv_bfloat16* __restrict__ y, int S,
                                      int K, int H, const unsigned long long* done_flags, int world,
                                      const unsigned long long* epoch_ptr, unsigned long long limit_ns,
                                      unsigned long long* status, const SwapCommitArgs commit) {
  const unsigned long long epoch = step_epoch(epoch_ptr, false);
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(status, TR_REDUCE);
  if (!block_wait_all(done_flags, world, epoch, limit_ns, status, WAIT_COMBINE)) return;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(status, TR_REDUCE_GO);
  const int vec_per_row = H / 8;
  const size_t total = (size_t)S * vec_per_row;
  const bool dead = status[ST_VIOLATION] != 0ull;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (!dead) {
      // eight independent 16-byte loads in flight per thread, then the fp32 adds in slot order
      for (int k0 = 0; k0 < K; k0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (k0 + q < K) raw[q] = reinterpret_cast<const uint4*>(panel + ((size_t)t * K + k0 + q) * H)[v];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (k0 + q < K) {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
#pragma unroll
            for (int z = 0; z < 4; ++z) {
              const float2 f = __bfloat1622float2(h2[z]);
              acc[2 * z] += f.x;
              acc[2 * z + 1] += f.y;
            }
          }
        }
      }
    }
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(y + t * H)[v] = out;
  }
  if (threadIdx.x == 0) trace_mark_max(status, TR_REDUCE_END);
  // every rank's combine GEMM has finished (the wait above), so nobody reads this rank's old slot contents any more:
  // the experts that arrived this step move from staging into their slots
  swap_commit(commit);
  if (threadIdx.x == 0) trace_mark_max(status, TR_RING + 16 + (int)(epoch & 15));
}

}  // namespace zepp
