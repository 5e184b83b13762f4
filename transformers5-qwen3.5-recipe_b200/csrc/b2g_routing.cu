// Router top-k, routing plan (stable counting sort + expert histogram), token permute / un-permute
// and SwiGLU: the HBM-bound byte/index kernels of the grouped path.  No atomics on outputs, so every
// result is bitwise reproducible from run to run.
#include "b2g_common.cuh"

namespace b2g {
namespace {

constexpr int kExperts = 256;

// ---------------------------------------------------------------------------------------------
// Router top-k: one warp per token row.  Lane l holds experts j*32+l (j = 0..7), so the eight loads
// of a warp are each one coalesced line.  Keys are (order-preserving score bits << 16) | (256 - id):
// the largest key is the best score and, among equal scores, the smallest expert id.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t b = __float_as_uint(f);
  return b ^ ((b & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
}

template <bool kFp32, bool kSqrtSoftplus>
__global__ void __launch_bounds__(256) router_topk_kernel(const void* __restrict__ logits, const float* __restrict__ bias,
                                                          int64_t* __restrict__ indices, int64_t T, int top_k) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t t = warp; t < T; t += nwarps) {
    unsigned long long key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = j * 32 + lane;
      float s;
      if (kFp32) s = static_cast<const float*>(logits)[t * kExperts + e];
      else s = __bfloat162float(static_cast<const __nv_bfloat16*>(logits)[t * kExperts + e]);
      if (kSqrtSoftplus) {
        const float sp = fmaxf(s, 0.0f) + logf(1.0f + expf(-fabsf(s)));
        s = sqrtf(sp);
        if (bias) s += bias[e];
      }
      key[j] = (static_cast<unsigned long long>(ordered_bits(s)) << 16) | static_cast<unsigned long long>(kExperts - e);
    }
    for (int r = 0; r < top_k; ++r) {
      unsigned long long best = key[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) best = key[j] > best ? key[j] : best;
      unsigned long long all = best;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xFFFFFFFFu, all, off);
        all = o > all ? o : all;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (key[j] == all) key[j] = 0;  // keys are unique (they embed the expert id)
      if (lane == 0) indices[t * top_k + r] = kExperts - static_cast<int64_t>(all & 0xFFFFull);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Routing plan.  Three passes over the flat id array, split into chunks of kChunk ids handled by one
// warp each so that ranks inside a chunk can be assigned in order (stable):
//   1. per-chunk histogram                       -> ws[chunk][E]
//   2. per-expert exclusive scan over chunks     -> ws = rows of that expert in earlier chunks; sizes, then offsets
//   3. per-chunk ordered scatter                 -> sorted_expert, perm, inv_perm
// ---------------------------------------------------------------------------------------------
constexpr int kChunk = 512;

template <bool kIdx64>
__device__ __forceinline__ int load_id(const void* p, int64_t i) {
  return kIdx64 ? static_cast<int>(static_cast<const int64_t*>(p)[i]) : static_cast<const int32_t*>(p)[i];
}

template <bool kIdx64>
__global__ void __launch_bounds__(256) plan_hist_kernel(const void* __restrict__ ids, int64_t R, int E, int32_t* __restrict__ ws,
                                                        int* __restrict__ status) {
  extern __shared__ int32_t sh[];  // [warps][E]
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* cnt = sh + warp_in_block * E;
  const int64_t chunk = blockIdx.x * (int64_t)(blockDim.x >> 5) + warp_in_block;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t begin = chunk * kChunk;
  if (begin < R) {
    const int64_t end = begin + kChunk < R ? begin + kChunk : R;
    for (int64_t i = begin + lane; i < end; i += 32) {
      const int e = load_id<kIdx64>(ids, i);
      if (e < 0 || e >= E) {              // not counted, not placed: reported through the status word
        if (status) atomicCAS(status, 0, 903);
        continue;
      }
      atomicAdd(&cnt[e], 1);  // shared-memory counter private to this warp: order does not matter
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) ws[chunk * E + e] = cnt[e];
  }
}

// One warp per expert: exclusive scan of that expert's per-chunk counts (32 chunks per step, shuffle scan).
__global__ void __launch_bounds__(256) plan_scan_kernel(int32_t* __restrict__ ws, int64_t nchunks, int E, int32_t* __restrict__ sizes) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= E) return;
  int32_t run = 0;
  for (int64_t c0 = 0; c0 < nchunks; c0 += 32) {
    const int64_t c = c0 + lane;
    const int32_t v = c < nchunks ? ws[c * E + e] : 0;
    int32_t incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int32_t o = __shfl_up_sync(0xFFFFFFFFu, incl, off);
      if (lane >= off) incl += o;
    }
    if (c < nchunks) ws[c * E + e] = run + incl - v;
    run += __shfl_sync(0xFFFFFFFFu, incl, 31);
  }
  if (lane == 0) sizes[e] = run;
}

// Cumulative ends over the experts (E <= 1024), one block.
__global__ void __launch_bounds__(1024) plan_offsets_kernel(const int32_t* __restrict__ sizes, int E, int32_t* __restrict__ offsets) {
  __shared__ int32_t tot[1024];
  const int e = threadIdx.x;
  tot[e] = e < E ? sizes[e] : 0;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t add = e >= off ? tot[e - off] : 0;
    __syncthreads();
    tot[e] += add;
    __syncthreads();
  }
  if (e < E) offsets[e] = tot[e];
}

template <bool kIdx64>
__global__ void __launch_bounds__(256) plan_scatter_kernel(const void* __restrict__ ids, int64_t R, int E,
                                                           const int32_t* __restrict__ ws, const int32_t* __restrict__ sizes,
                                                           const int32_t* __restrict__ offsets, int64_t* __restrict__ sorted_expert,
                                                           int64_t* __restrict__ perm, int64_t* __restrict__ inv_perm) {
  extern __shared__ int32_t sh[];
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* next = sh + warp_in_block * E;
  const int64_t chunk = blockIdx.x * (int64_t)(blockDim.x >> 5) + warp_in_block;
  const int64_t begin = chunk * kChunk;
  if (begin >= R) return;
  for (int e = lane; e < E; e += 32) next[e] = ws[chunk * E + e] + offsets[e] - sizes[e];  // chunk prefix + first slot of the expert
  __syncwarp();
  const int64_t end = begin + kChunk < R ? begin + kChunk : R;
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t i = base + lane;
    const bool live = i < end;
    int e = live ? load_id<kIdx64>(ids, i) : -1 - lane;  // dead lanes get unique negative ids
    if (live && (e < 0 || e >= E)) e = -1 - lane;         // out-of-range ids were flagged by pass 1
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    const int leader = __ffs(peers) - 1;
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int32_t first = 0;
    if (e >= 0 && lane == leader) {
      first = next[e];
      next[e] = first + __popc(peers);
    }
    first = __shfl_sync(0xFFFFFFFFu, first, leader);
    __syncwarp();
    if (e >= 0) {
      const int64_t pos = first + rank;
      sorted_expert[pos] = e;
      perm[pos] = i;
      inv_perm[i] = pos;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Permute / un-permute.  Rows are H bf16 wide; a thread moves 8 values (16 bytes) at a time.
// ---------------------------------------------------------------------------------------------
// One warp per destination row, up to eight 16-byte loads in flight per lane.
__global__ void __launch_bounds__(256) gather_kernel(const uint4* __restrict__ hidden, const int64_t* __restrict__ perm,
                                                     uint4* __restrict__ sel, int64_t R, int top_k, int vec_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t s = warp; s < R; s += nwarps) {
    const int64_t tok = perm[s] / top_k;
    const uint4* src = hidden + tok * vec_per_row;
    uint4* dst = sel + s * vec_per_row;
    for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
      uint4 buf[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int v = v0 + lane + 32 * i;
        if (v < vec_per_row) buf[i] = src[v];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int v = v0 + lane + 32 * i;
        if (v < vec_per_row) dst[v] = buf[i];
      }
    }
  }
}

// acc += g on eight bf16 values, each sum rounded to bf16 (round to nearest even): the packed bf16 add is the exactly rounded
// sum, which is what adding in fp32 and rounding gives for bf16 operands (the fp32 sum is exact unless the exponents are more
// than 16 apart, and then both forms return the larger operand).
__device__ __forceinline__ void add_round8(uint4& acc, const uint4 g) {
  const __nv_bfloat162* gv = reinterpret_cast<const __nv_bfloat162*>(&g);
  __nv_bfloat162* av = reinterpret_cast<__nv_bfloat162*>(&acc);
#pragma unroll
  for (int i = 0; i < 4; ++i) av[i] = __hadd2(av[i], gv[i]);
}

__global__ void __launch_bounds__(256) gather_bwd_kernel(const uint4* __restrict__ grad_sel, const int64_t* __restrict__ inv,
                                                         uint4* __restrict__ grad_hidden, int64_t T, int top_k, int vec_per_row) {
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {
    int64_t pos[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pos[j] = j < top_k ? inv[t * top_k + j] : INT64_MAX;
    // ascending order of sorted position (8-element insertion network; top_k <= 8)
#pragma unroll
    for (int a = 1; a < 8; ++a)
#pragma unroll
      for (int b = a; b > 0; --b)
        if (pos[b] < pos[b - 1]) { const int64_t x = pos[b]; pos[b] = pos[b - 1]; pos[b - 1] = x; }
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 rows[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < top_k) rows[j] = grad_sel[pos[j] * vec_per_row + v];
      uint4 acc = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < top_k) add_round8(acc, rows[j]);
      grad_hidden[t * vec_per_row + v] = acc;
    }
  }
}

template <bool kW32>
__device__ __forceinline__ float load_weight_bf16(const void* w, int64_t i) {
  if (kW32) return dev::round_bf16(static_cast<const float*>(w)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]);
}

template <bool kW32>
__global__ void __launch_bounds__(256) combine_kernel(const uint4* __restrict__ expert_out, const void* __restrict__ weights,
                                                      const int64_t* __restrict__ inv, uint4* __restrict__ out, int64_t T,
                                                      int top_k, int vec_per_row) {
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {
    int64_t pos[8];
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pos[j] = j < top_k ? inv[t * top_k + j] : 0;
      w[j] = j < top_k ? load_weight_bf16<kW32>(weights, t * top_k + j) : 0.f;
    }
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 rows[8];                              // all of a token's rows in flight before the first FMA
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < top_k) rows[j] = expert_out[pos[j] * vec_per_row + v];
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < top_k) {
          const uint4 g = rows[j];
          const uint32_t q[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(dev::bf16_lo(q[i]), w[j], acc[2 * i]);
            acc[2 * i + 1] = fmaf(dev::bf16_hi(q[i]), w[j], acc[2 * i + 1]);
          }
        }
      }
      uint4 o;
      o.x = dev::pack_bf16(acc[0], acc[1]); o.y = dev::pack_bf16(acc[2], acc[3]);
      o.z = dev::pack_bf16(acc[4], acc[5]); o.w = dev::pack_bf16(acc[6], acc[7]);
      out[t * vec_per_row + v] = o;
    }
  }
}

// One warp per routed row: no block-wide barrier, eight independent rows in flight per block.
template <bool kW32>
__global__ void __launch_bounds__(256) combine_bwd_kernel(const uint4* __restrict__ expert_out, const void* __restrict__ weights,
                                                          const int64_t* __restrict__ perm, const uint4* __restrict__ grad_final,
                                                          uint4* __restrict__ grad_out, void* __restrict__ grad_w, int64_t R,
                                                          int top_k, int vec_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t s = warp; s < R; s += nwarps) {
    const int64_t route = perm[s];
    const int64_t tok = route / top_k;
    const float w = load_weight_bf16<kW32>(weights, route);
    float dot = 0.f;
    for (int v0 = lane; v0 < vec_per_row; v0 += 128) {   // four vectors of each operand in flight per lane
      uint4 gs[4], ys[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + 32 * u;
        if (v < vec_per_row) { gs[u] = grad_final[tok * vec_per_row + v]; ys[u] = expert_out[s * vec_per_row + v]; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = v0 + 32 * u;
        if (v >= vec_per_row) break;
        const uint32_t gq[4] = {gs[u].x, gs[u].y, gs[u].z, gs[u].w}, yq[4] = {ys[u].x, ys[u].y, ys[u].z, ys[u].w};
        uint32_t oq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float g0 = dev::bf16_lo(gq[i]), g1 = dev::bf16_hi(gq[i]);
          oq[i] = dev::pack_bf16(__fmul_rn(g0, w), __fmul_rn(g1, w));
          dot = fmaf(g0, dev::bf16_lo(yq[i]), dot);
          dot = fmaf(g1, dev::bf16_hi(yq[i]), dot);
        }
        grad_out[s * vec_per_row + v] = make_uint4(oq[0], oq[1], oq[2], oq[3]);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
    if (lane == 0) {
      if (kW32) static_cast<float*>(grad_w)[route] = dot;
      else static_cast<__nv_bfloat16*>(grad_w)[route] = __float2bfloat16_rn(dot);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU, rounding to bf16 at the same points as a bf16 `silu(g) * u` in PyTorch.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// `row_begin` / `row_end` (device, nullable): the rows [*row_begin, *row_end) of `pairs_per_row` bf16 pairs each are the only
// ones that hold data (one expert group inside an expert-parallel receive buffer); nothing else is read or written.
__device__ __forceinline__ void live_pairs(int64_t npairs, const int32_t* row_begin, const int32_t* row_end, int64_t pairs_per_row,
                                           int64_t& first, int64_t& last) {
  first = row_begin ? static_cast<int64_t>(*row_begin) * pairs_per_row : 0;
  last = row_end ? static_cast<int64_t>(*row_end) * pairs_per_row : npairs;
  if (first < 0) first = 0;
  if (last > npairs) last = npairs;
}

__device__ __forceinline__ uint32_t swiglu_fwd_pair(uint32_t g2, uint32_t u2, float limit) {
  float g[2] = {dev::bf16_lo(g2), dev::bf16_hi(g2)}, u[2] = {dev::bf16_lo(u2), dev::bf16_hi(u2)}, o[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (limit > 0.f) { g[k] = fminf(g[k], limit); u[k] = fminf(fmaxf(u[k], -limit), limit); }
    const float act = dev::round_bf16(g[k] * sigmoidf_(g[k]));
    o[k] = act * u[k];
  }
  return dev::pack_bf16(o[0], o[1]);
}

__device__ __forceinline__ void swiglu_bwd_pair(uint32_t g2, uint32_t u2, uint32_t d2, float limit, uint32_t& dg2, uint32_t& du2) {
  const float g[2] = {dev::bf16_lo(g2), dev::bf16_hi(g2)}, u[2] = {dev::bf16_lo(u2), dev::bf16_hi(u2)};
  const float d[2] = {dev::bf16_lo(d2), dev::bf16_hi(d2)};
  float og[2], ou[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    float gc = g[k], uc = u[k];
    bool g_pass = true, u_pass = true;
    if (limit > 0.f) {
      g_pass = g[k] <= limit; u_pass = (u[k] >= -limit) && (u[k] <= limit);
      gc = fminf(gc, limit); uc = fminf(fmaxf(uc, -limit), limit);
    }
    const float sig = sigmoidf_(gc);
    const float act = dev::round_bf16(gc * sig);
    const float dact = dev::round_bf16(d[k] * uc);
    ou[k] = u_pass ? d[k] * act : 0.f;
    og[k] = g_pass ? dact * (sig * (1.0f + gc * (1.0f - sig))) : 0.f;
  }
  dg2 = dev::pack_bf16(og[0], og[1]);
  du2 = dev::pack_bf16(ou[0], ou[1]);
}

// kVec: every thread moves 16 bytes (four bf16 pairs) per operand and step; the host picks it when the live range and the
// pointers allow it (they do for every expert width in use), else the pair-at-a-time form.
template <bool kVec>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint32_t* __restrict__ gate, const uint32_t* __restrict__ up,
                                                         uint32_t* __restrict__ z, int64_t npairs, float limit,
                                                         const int32_t* __restrict__ row_begin, const int32_t* __restrict__ row_end,
                                                         int64_t pairs_per_row) {
  int64_t first, last;
  live_pairs(npairs, row_begin, row_end, pairs_per_row, first, last);
  if constexpr (kVec) {
    const uint4* g4 = reinterpret_cast<const uint4*>(gate);
    const uint4* u4 = reinterpret_cast<const uint4*>(up);
    uint4* z4 = reinterpret_cast<uint4*>(z);
    for (int64_t i = first / 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < last / 4; i += (int64_t)gridDim.x * blockDim.x) {
      const uint4 g = g4[i], u = u4[i];
      z4[i] = make_uint4(swiglu_fwd_pair(g.x, u.x, limit), swiglu_fwd_pair(g.y, u.y, limit), swiglu_fwd_pair(g.z, u.z, limit),
                         swiglu_fwd_pair(g.w, u.w, limit));
    }
  } else {
    for (int64_t i = first + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < last; i += (int64_t)gridDim.x * blockDim.x)
      z[i] = swiglu_fwd_pair(gate[i], up[i], limit);
  }
}

template <bool kVec>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint32_t* __restrict__ gate, const uint32_t* __restrict__ up,
                                                         const uint32_t* __restrict__ dz, uint32_t* __restrict__ dgate,
                                                         uint32_t* __restrict__ dup, int64_t npairs, float limit,
                                                         const int32_t* __restrict__ row_begin, const int32_t* __restrict__ row_end,
                                                         int64_t pairs_per_row) {
  int64_t first, last;
  live_pairs(npairs, row_begin, row_end, pairs_per_row, first, last);
  if constexpr (kVec) {
    const uint4* g4 = reinterpret_cast<const uint4*>(gate);
    const uint4* u4 = reinterpret_cast<const uint4*>(up);
    const uint4* d4 = reinterpret_cast<const uint4*>(dz);
    uint4* dg4 = reinterpret_cast<uint4*>(dgate);
    uint4* du4 = reinterpret_cast<uint4*>(dup);
    for (int64_t i = first / 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < last / 4; i += (int64_t)gridDim.x * blockDim.x) {
      const uint4 g = g4[i], u = u4[i], d = d4[i];
      uint4 og, ou;
      swiglu_bwd_pair(g.x, u.x, d.x, limit, og.x, ou.x);
      swiglu_bwd_pair(g.y, u.y, d.y, limit, og.y, ou.y);
      swiglu_bwd_pair(g.z, u.z, d.z, limit, og.z, ou.z);
      swiglu_bwd_pair(g.w, u.w, d.w, limit, og.w, ou.w);
      dg4[i] = og;
      du4[i] = ou;
    }
  } else {
    for (int64_t i = first + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < last; i += (int64_t)gridDim.x * blockDim.x) {
      uint32_t og, ou;
      swiglu_bwd_pair(gate[i], up[i], dz[i], limit, og, ou);
      dgate[i] = og;
      dup[i] = ou;
    }
  }
}

inline int row_grid(int64_t rows) {
  const int64_t cap = (int64_t)sm_count() * 8;
  return static_cast<int>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

}  // namespace
}  // namespace b2g

using namespace b2g;

extern "C" int b2g_router_topk(const void* logits, int logits_dtype, const float* bias, int score_fn, int64_t* indices,
                               int64_t T, int E, int top_k, void* stream) {
  B2G_REQUIRE(E == kExperts, "router top-k supports exactly 256 experts, got %d", E);
  B2G_REQUIRE(top_k >= 1 && top_k <= 8, "top_k=%d outside 1..8", top_k);
  B2G_REQUIRE(logits_dtype == 0 || logits_dtype == 1, "logits_dtype must be 0 (bf16) or 1 (fp32)");
  B2G_REQUIRE(score_fn == 0 || score_fn == 1, "score_fn must be 0 (identity) or 1 (sqrtsoftplus)");
  B2G_REQUIRE(score_fn == 1 || bias == nullptr, "a correction bias needs sqrtsoftplus scoring");
  if (T == 0) return 0;
  B2G_REQUIRE(T > 0 && logits && indices, "bad token count or null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t want = (T + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 8;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  if (logits_dtype == 1) {
    if (score_fn) router_topk_kernel<true, true><<<blocks, 256, 0, s>>>(logits, bias, indices, T, top_k);
    else router_topk_kernel<true, false><<<blocks, 256, 0, s>>>(logits, bias, indices, T, top_k);
  } else {
    if (score_fn) router_topk_kernel<false, true><<<blocks, 256, 0, s>>>(logits, bias, indices, T, top_k);
    else router_topk_kernel<false, false><<<blocks, 256, 0, s>>>(logits, bias, indices, T, top_k);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int64_t b2g_route_plan_workspace_bytes(int64_t R, int E) {
  const int64_t nchunks = (R + kChunk - 1) / kChunk;
  return (nchunks * E + 4) * (int64_t)sizeof(int32_t);
}

extern "C" int b2g_route_plan(const void* topk_idx, int idx_dtype, int64_t T, int top_k, int E, int64_t* sorted_expert,
                              int64_t* perm, int64_t* inv_perm, int32_t* group_sizes, int32_t* offsets, void* workspace,
                              int64_t workspace_bytes, int* status, void* stream) {
  B2G_REQUIRE(idx_dtype == 0 || idx_dtype == 1, "idx_dtype must be 0 (int32) or 1 (int64)");
  B2G_REQUIRE(E >= 1 && E <= 1024, "E=%d outside 1..1024", E);
  B2G_REQUIRE(T >= 0 && top_k >= 1, "bad T/top_k");
  const int64_t R = T * top_k;
  B2G_REQUIRE(R < (1ll << 31), "too many routes");
  B2G_REQUIRE(workspace_bytes >= b2g_route_plan_workspace_bytes(R, E), "workspace too small: %lld < %lld",
              (long long)workspace_bytes, (long long)b2g_route_plan_workspace_bytes(R, E));
  B2G_REQUIRE(group_sizes && offsets && workspace, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t nchunks = (R + kChunk - 1) / kChunk;
  int32_t* ws = static_cast<int32_t*>(workspace);
  const int warps = 8;
  const size_t smem = (size_t)warps * E * sizeof(int32_t);
  const int blocks = static_cast<int>((nchunks + warps - 1) / warps);
  if (R > 0) {
    B2G_REQUIRE(topk_idx && sorted_expert && perm && inv_perm, "null pointer");
    if (idx_dtype) plan_hist_kernel<true><<<blocks, warps * 32, smem, s>>>(topk_idx, R, E, ws, status);
    else plan_hist_kernel<false><<<blocks, warps * 32, smem, s>>>(topk_idx, R, E, ws, status);
  }
  plan_scan_kernel<<<(E + 7) / 8, 256, 0, s>>>(ws, nchunks, E, group_sizes);
  plan_offsets_kernel<<<1, 1024, 0, s>>>(group_sizes, E, offsets);
  if (R > 0) {
    if (idx_dtype) plan_scatter_kernel<true><<<blocks, warps * 32, smem, s>>>(topk_idx, R, E, ws, group_sizes, offsets, sorted_expert, perm, inv_perm);
    else plan_scatter_kernel<false><<<blocks, warps * 32, smem, s>>>(topk_idx, R, E, ws, group_sizes, offsets, sorted_expert, perm, inv_perm);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

#define B2G_ROW_ARGS_OK(H)                                                                     \
  B2G_REQUIRE((H) > 0 && (H) % 8 == 0, "hidden width %d must be a positive multiple of 8", (H)); \
  B2G_REQUIRE(top_k >= 1 && top_k <= 8, "top_k=%d outside 1..8", top_k)

extern "C" int b2g_route_gather(const void* hidden, const int64_t* perm, void* selected, int64_t T, int top_k, int H, void* stream) {
  B2G_ROW_ARGS_OK(H);
  const int64_t R = T * top_k;
  if (R == 0) return 0;
  B2G_REQUIRE(hidden && perm && selected && aligned16(hidden) && aligned16(selected), "null or misaligned pointer");
  gather_kernel<<<row_grid((R + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(hidden), perm,
                                                                            static_cast<uint4*>(selected), R, top_k, H / 8);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_route_gather_bwd(const void* grad_selected, const int64_t* inv_perm, void* grad_hidden, int64_t T, int top_k,
                                    int H, void* stream) {
  B2G_ROW_ARGS_OK(H);
  if (T == 0) return 0;
  B2G_REQUIRE(grad_selected && inv_perm && grad_hidden && aligned16(grad_selected) && aligned16(grad_hidden),
              "null or misaligned pointer");
  gather_bwd_kernel<<<row_grid(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(grad_selected), inv_perm, static_cast<uint4*>(grad_hidden), T, top_k, H / 8);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_route_combine(const void* expert_out, const void* weights, int w_dtype, const int64_t* inv_perm, void* out,
                                 int64_t T, int top_k, int H, void* stream) {
  B2G_ROW_ARGS_OK(H);
  B2G_REQUIRE(w_dtype == 0 || w_dtype == 1, "w_dtype must be 0 (bf16) or 1 (fp32)");
  if (T == 0) return 0;
  B2G_REQUIRE(expert_out && weights && inv_perm && out && aligned16(expert_out) && aligned16(out), "null or misaligned pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w_dtype) combine_kernel<true><<<row_grid(T), 256, 0, s>>>(static_cast<const uint4*>(expert_out), weights, inv_perm,
                                                                static_cast<uint4*>(out), T, top_k, H / 8);
  else combine_kernel<false><<<row_grid(T), 256, 0, s>>>(static_cast<const uint4*>(expert_out), weights, inv_perm,
                                                         static_cast<uint4*>(out), T, top_k, H / 8);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_route_combine_bwd(const void* expert_out, const void* weights, int w_dtype, const int64_t* perm,
                                     const void* grad_final, void* grad_expert_out, void* grad_weights, int64_t T, int top_k,
                                     int H, void* stream) {
  B2G_ROW_ARGS_OK(H);
  B2G_REQUIRE(w_dtype == 0 || w_dtype == 1, "w_dtype must be 0 (bf16) or 1 (fp32)");
  const int64_t R = T * top_k;
  if (R == 0) return 0;
  B2G_REQUIRE(expert_out && weights && perm && grad_final && grad_expert_out && grad_weights, "null pointer");
  B2G_REQUIRE(aligned16(expert_out) && aligned16(grad_final) && aligned16(grad_expert_out), "misaligned pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w_dtype) combine_bwd_kernel<true><<<row_grid((R + 7) / 8), 256, 0, s>>>(static_cast<const uint4*>(expert_out), weights, perm,
                                                                    static_cast<const uint4*>(grad_final),
                                                                    static_cast<uint4*>(grad_expert_out), grad_weights, R, top_k, H / 8);
  else combine_bwd_kernel<false><<<row_grid((R + 7) / 8), 256, 0, s>>>(static_cast<const uint4*>(expert_out), weights, perm,
                                                             static_cast<const uint4*>(grad_final),
                                                             static_cast<uint4*>(grad_expert_out), grad_weights, R, top_k, H / 8);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_swiglu_fwd(const void* gate, const void* up, void* z, int64_t n, float limit, const int32_t* row_begin,
                              const int32_t* row_end, int64_t cols, void* stream) {
  B2G_REQUIRE(n >= 0 && n % 2 == 0, "element count must be even");
  B2G_REQUIRE((row_begin == nullptr && row_end == nullptr) || (cols > 0 && cols % 2 == 0 && n % cols == 0),
              "a row range needs an even row width that divides n");
  if (n == 0) return 0;
  B2G_REQUIRE(gate && up && z, "null pointer");
  const int64_t pairs = n / 2;
  const bool vec = pairs % 4 == 0 && aligned16(gate) && aligned16(up) && aligned16(z) && (row_begin == nullptr && row_end == nullptr ? true : cols % 8 == 0);
  const int64_t want = ((vec ? pairs / 4 : pairs) + 255) / 256, cap = (int64_t)sm_count() * 16;
  const int grid = (int)(want < cap ? want : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (vec) {
    B2G_KERNEL_MAX_SHARED(swiglu_fwd_kernel<true>);
    swiglu_fwd_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(gate), static_cast<const uint32_t*>(up), static_cast<uint32_t*>(z),
                                                  pairs, limit, row_begin, row_end, cols / 2);
  } else {
    B2G_KERNEL_MAX_SHARED(swiglu_fwd_kernel<false>);
    swiglu_fwd_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(gate), static_cast<const uint32_t*>(up), static_cast<uint32_t*>(z),
                                                   pairs, limit, row_begin, row_end, cols / 2);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_swiglu_bwd(const void* gate, const void* up, const void* dz, void* dgate, void* dup, int64_t n, float limit,
                              const int32_t* row_begin, const int32_t* row_end, int64_t cols, void* stream) {
  B2G_REQUIRE(n >= 0 && n % 2 == 0, "element count must be even");
  B2G_REQUIRE((row_begin == nullptr && row_end == nullptr) || (cols > 0 && cols % 2 == 0 && n % cols == 0),
              "a row range needs an even row width that divides n");
  if (n == 0) return 0;
  B2G_REQUIRE(gate && up && dz && dgate && dup, "null pointer");
  const int64_t pairs = n / 2;
  const bool vec = pairs % 4 == 0 && aligned16(gate) && aligned16(up) && aligned16(dz) && aligned16(dgate) && aligned16(dup) &&
                   (row_begin == nullptr && row_end == nullptr ? true : cols % 8 == 0);
  const int64_t want = ((vec ? pairs / 4 : pairs) + 255) / 256, cap = (int64_t)sm_count() * 16;
  const int grid = (int)(want < cap ? want : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (vec) {
    B2G_KERNEL_MAX_SHARED(swiglu_bwd_kernel<true>);
    swiglu_bwd_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(gate), static_cast<const uint32_t*>(up),
                                                  static_cast<const uint32_t*>(dz), static_cast<uint32_t*>(dgate),
                                                  static_cast<uint32_t*>(dup), pairs, limit, row_begin, row_end, cols / 2);
  } else {
    B2G_KERNEL_MAX_SHARED(swiglu_bwd_kernel<false>);
    swiglu_bwd_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(gate), static_cast<const uint32_t*>(up),
                                                   static_cast<const uint32_t*>(dz), static_cast<uint32_t*>(dgate),
                                                   static_cast<uint32_t*>(dup), pairs, limit, row_begin, row_end, cols / 2);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}
