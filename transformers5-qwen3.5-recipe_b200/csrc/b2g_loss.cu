// Cross-entropy over a chunk of bf16 logits, in place: each row's loss goes to a float array and the logits are
// overwritten by their cotangent (softmax - onehot) * scale, rounded to bf16, ready to be multiplied back through the
// packed LM head.  One CTA per row; two passes over the row (online max / sum of exponentials, then the gradient), the
// second of which is served by L2 for the chunk sizes this is used with (512 rows x 129280 logits = 132 MB is the
// largest; 256 rows fit entirely).  HBM-bound: 2 B read + 2 B written per logit, plus the L2 re-read.
#include "b2g_common.cuh"

namespace b2g {
namespace loss {

constexpr int kThreads = 1024;

struct RowStat { float m, d; float best; int best_i; };

__device__ __forceinline__ void merge(RowStat& a, const RowStat& b) {
  const float m = fmaxf(a.m, b.m);
  // exp(-inf - -inf) must not appear: a side that saw nothing has d == 0 and contributes nothing
  a.d = (a.d > 0.f ? a.d * __expf(a.m - m) : 0.f) + (b.d > 0.f ? b.d * __expf(b.m - m) : 0.f);
  a.m = m;
  if (b.best > a.best || (b.best == a.best && b.best_i < a.best_i)) { a.best = b.best; a.best_i = b.best_i; }
}

__device__ __forceinline__ void visit(RowStat& s, float x, int i) {
  if (x > s.m) { s.d = s.d * __expf(s.m - x) + 1.f; s.m = x; }
  else s.d += __expf(x - s.m);
  if (x > s.best) { s.best = x; s.best_i = i; }   // ascending i within a thread: the first maximum is kept
}

// `kVec`: rows are 16-byte aligned and V % 8 == 0 (vector path); otherwise element accesses.
template <bool kVec>
__global__ void __launch_bounds__(kThreads) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, int64_t ld, const int64_t* __restrict__ target,
                                                                 float* __restrict__ loss, int64_t* __restrict__ predicted,
                                                                 float* __restrict__ correct, int V, int64_t ignore_index,
                                                                 const int64_t* __restrict__ count, int mean, int* status) {
  __shared__ RowStat part[kThreads / 32];
  __shared__ RowStat total;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __nv_bfloat16* x = logits + (int64_t)row * ld;
  const int64_t y = target[row];
  const bool ignored = y == ignore_index;
  const bool bad = !ignored && (y < 0 || y >= V);
  if (bad && threadIdx.x == 0 && status) atomicCAS(status, 0, 902);   // label outside the vocabulary: reported, row treated as ignored

  RowStat s{-INFINITY, 0.f, -INFINITY, 0x7fffffff};
  if (kVec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int v = threadIdx.x; v < V / 8; v += kThreads) {
      const uint4 q = xv[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        visit(s, dev::bf16_lo(w[j]), 8 * v + 2 * j);
        visit(s, dev::bf16_hi(w[j]), 8 * v + 2 * j + 1);
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += kThreads) visit(s, __bfloat162float(x[i]), i);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    RowStat o;
    o.m = __shfl_xor_sync(0xffffffffu, s.m, off);
    o.d = __shfl_xor_sync(0xffffffffu, s.d, off);
    o.best = __shfl_xor_sync(0xffffffffu, s.best, off);
    o.best_i = __shfl_xor_sync(0xffffffffu, s.best_i, off);
    merge(s, o);
  }
  if (lane == 0) part[warp] = s;
  __syncthreads();
  if (warp == 0) {
    RowStat t = lane < kThreads / 32 ? part[lane] : RowStat{-INFINITY, 0.f, -INFINITY, 0x7fffffff};
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      RowStat o;
      o.m = __shfl_xor_sync(0xffffffffu, t.m, off);
      o.d = __shfl_xor_sync(0xffffffffu, t.d, off);
      o.best = __shfl_xor_sync(0xffffffffu, t.best, off);
      o.best_i = __shfl_xor_sync(0xffffffffu, t.best_i, off);
      merge(t, o);
    }
    if (lane == 0) total = t;
  }
  __syncthreads();
  const RowStat t = total;
  const bool live = !ignored && !bad;
  float scale = 1.f;
  if (mean) {
    const int64_t n = *count;
    scale = n > 0 ? 1.f / static_cast<float>(n) : 0.f;
  }
  if (threadIdx.x == 0) {
    const float xy = live ? __bfloat162float(x[y]) : 0.f;
    loss[row] = live ? (t.m + __logf(t.d) - xy) * scale : 0.f;
    if (predicted) predicted[row] = live ? t.best_i : -1;
    if (correct) correct[row] = (live && t.best_i == y) ? 1.f : 0.f;
  }
  __syncthreads();   // x[y] is read before anyone overwrites it
  const float inv_d = live ? scale / t.d : 0.f;
  const int yi = live ? static_cast<int>(y) : -1;
  if (kVec) {
    uint4* xv = reinterpret_cast<uint4*>(x);
    for (int v = threadIdx.x; v < V / 8; v += kThreads) {
      const uint4 q = xv[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i0 = 8 * v + 2 * j;
        float g0 = __expf(dev::bf16_lo(w[j]) - t.m) * inv_d, g1 = __expf(dev::bf16_hi(w[j]) - t.m) * inv_d;
        if (i0 == yi) g0 -= scale;
        if (i0 + 1 == yi) g1 -= scale;
        o[j] = dev::pack_bf16(live ? g0 : 0.f, live ? g1 : 0.f);
      }
      xv[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += kThreads) {
      float g = __expf(__bfloat162float(x[i]) - t.m) * inv_d;
      if (i == yi) g -= scale;
      x[i] = __float2bfloat16_rn(live ? g : 0.f);
    }
  }
}

}  // namespace loss
}  // namespace b2g

using namespace b2g;

extern "C" int b2g_cross_entropy_inplace(void* logits, int64_t ld, const int64_t* target, float* loss, int64_t* predicted, float* correct,
                                         int64_t rows, int64_t V, int64_t ignore_index, const int64_t* count, int mean, int* status,
                                         void* stream) {
  B2G_REQUIRE(rows >= 0 && V >= 1 && V < (1ll << 31) && ld >= V, "cross_entropy: bad shape rows=%lld V=%lld ld=%lld", (long long)rows,
              (long long)V, (long long)ld);
  if (rows == 0) return 0;
  B2G_REQUIRE(logits && target && loss, "cross_entropy: null pointer");
  B2G_REQUIRE(!mean || count, "cross_entropy: mean reduction needs the device count of non-ignored targets");
  B2G_REQUIRE(rows < (1ll << 31), "cross_entropy: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* x = static_cast<__nv_bfloat16*>(logits);
  const bool vec = aligned16(logits) && ld % 8 == 0 && V % 8 == 0;
  if (vec)
    loss::cross_entropy_kernel<true><<<(int)rows, loss::kThreads, 0, s>>>(x, ld, target, loss, predicted, correct, (int)V, ignore_index, count,
                                                                          mean, status);
  else
    loss::cross_entropy_kernel<false><<<(int)rows, loss::kThreads, 0, s>>>(x, ld, target, loss, predicted, correct, (int)V, ignore_index,
                                                                           count, mean, status);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}
