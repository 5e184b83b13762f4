// LoRA rank-side products: the skinny projections (X.A^T, dY.B) and the factor gradients
// (contractions over the token rows).  Output widths are <= 16, so these kernels are bound by
// streaming X / dY once from HBM; tiles arrive through TMA (the projection with [r, C] weights, the
// dense factor gradient) or a cp.async pipeline (the rest) and the arithmetic is bf16 mma.sync with
// fp32 accumulation.  The same kernels serve the dense path (one weight) and the
// grouped path (one weight per expert segment).
#include "b2g_common.cuh"

#include <mutex>

namespace b2g {
namespace lora {

constexpr int kRankPad = B2G_LORA_PAD;  // 16

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // src-size 0 zero-fills the destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Row segment handled by one CTA.
struct Seg { int expert, row0, rows; };

// ------------------------------------------------------------------------------------------------
// Projection: P[rows,16] = X[rows,C] . W_e^T  (r <= 16 columns live, the rest zero)
// CTA = 4 warps x 16 rows; reduction in chunks of 128 columns, 4-stage cp.async ring.
// ------------------------------------------------------------------------------------------------
constexpr int kDownRows = 64, kDownBK = 128, kDownStages = 4, kDownStride = kDownBK * 2 + 16;  // 272-byte rows
constexpr int kDownXBytes = kDownRows * kDownStride, kDownWBytes = kRankPad * kDownStride;
constexpr int kDownStageBytes = kDownXBytes + kDownWBytes;

// Grouped: item = one 64-row slice of a tile of the schedule.  Dense: every CTA owns one contiguous range of
// `dense_rows` rows (the same byte count for every CTA, so that none runs a round longer than the others) and
// walks it in slices of 64; `item` is then blockIdx.x + slice * gridDim.x.
__device__ __forceinline__ Seg down_segment(const int4* tiles, int64_t m_total, int item, int dense_rows) {
  Seg s;
  if (tiles) {
    const int rows_per_tile = tiles[0].y;
    const int per = rows_per_tile / kDownRows;
    const int4 e = tiles[1 + item / per];
    const int sub = item % per;
    s.expert = e.x;
    s.row0 = e.y + sub * kDownRows;
    const int left = e.z - sub * kDownRows;
    s.rows = left < 0 ? 0 : (left < kDownRows ? left : kDownRows);
  } else {
    const int cta = item % gridDim.x, slice = item / gridDim.x;
    const int64_t first = (int64_t)cta * dense_rows + (int64_t)slice * kDownRows;
    int64_t end = (int64_t)(cta + 1) * dense_rows;
    if (end > m_total) end = m_total;
    const int64_t left = end - first;
    s.expert = 0;
    s.row0 = (int)first;
    s.rows = left < 0 ? 0 : (left < kDownRows ? (int)left : kDownRows);
  }
  return s;
}

// Each stage holds a [64 x 128] slice of X and the matching [16 x 128] slice of W^T (rank rows, reduction
// columns); both feed mma.sync through ldmatrix.  W given as [r, C] streams in with cp.async; W given as
// [C, r] is transposed on the way in (one reduction column per thread, registers as the staging buffer).
template <bool kWisCR>
__global__ void __launch_bounds__(128) lora_down_kernel(const __nv_bfloat16* __restrict__ x0, const __nv_bfloat16* __restrict__ x1,
                                                        const __nv_bfloat16* __restrict__ w, float scale, const int4* __restrict__ tiles,
                                                        __nv_bfloat16* __restrict__ out_plain, __nv_bfloat16* __restrict__ out_scaled,
                                                        int64_t m_total, int C, int r, int dense_rows) {
  extern __shared__ __align__(16) uint8_t sm[];
  const uint32_t sbase = dev::smem_u32(sm);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nseg = x1 ? 2 : 1;
  const int chunks = (C + kDownBK - 1) / kDownBK;
  const int total_items = tiles ? tiles[0].x * (tiles[0].y / kDownRows) : (int)gridDim.x * ((dense_rows + kDownRows - 1) / kDownRows);
  const int64_t w_per_expert = (int64_t)nseg * C * r;
  const int total_chunks = nseg * chunks;

  // rank rows >= r of every W stage stay zero for the whole kernel
  for (int i = threadIdx.x; i < kDownStages * kRankPad * (kDownStride / 4); i += blockDim.x) {
    const int st = i / (kRankPad * (kDownStride / 4)), rem = i - st * (kRankPad * (kDownStride / 4));
    reinterpret_cast<uint32_t*>(sm + st * kDownStageBytes + kDownXBytes)[rem] = 0u;
  }
  __syncthreads();

  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const Seg s = down_segment(tiles, m_total, item, dense_rows);
    if (s.rows <= 0) continue;
    const __nv_bfloat16* we = w + s.expert * w_per_expert;
    float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};

    auto issue_x = [&](int ch) {
      const int seg = ch / chunks, c0 = (ch - seg * chunks) * kDownBK;
      const __nv_bfloat16* xs = seg ? x1 : x0;
      const uint32_t dst = sbase + (ch % kDownStages) * kDownStageBytes;
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // 64 rows x 16 vectors of 16 bytes over 128 threads
        const int v = threadIdx.x + i * 128;
        const int row = v >> 4, vec = v & 15;
        const bool ok = row < s.rows && c0 + vec * 8 < C;  // zero-fill past the last row / column
        const __nv_bfloat16* src = xs + (int64_t)(s.row0 + (ok ? row : 0)) * C + (ok ? c0 + vec * 8 : 0);
        cp_async16(dst + row * kDownStride + vec * 16, src, ok);
      }
      if (!kWisCR) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // 16 rank rows x 16 vectors
          const int v = threadIdx.x + i * 128;
          const int row = v >> 4, vec = v & 15;
          const bool ok = row < r && c0 + vec * 8 < C;
          const __nv_bfloat16* src = we + (int64_t)(ok ? row : 0) * (nseg * C) + seg * C + (ok ? c0 + vec * 8 : 0);
          if (row < r) cp_async16(dst + kDownXBytes + row * kDownStride + vec * 16, src, ok);
        }
      }
    };
    // [C, r] layout: this thread's reduction column of chunk `ch` -> registers / registers -> stage
    unsigned short wv[kRankPad];
    auto load_w = [&](int ch) {
      const int seg = ch / chunks, k = (ch - seg * chunks) * kDownBK + threadIdx.x;
      const unsigned short* src = reinterpret_cast<const unsigned short*>(we) + ((int64_t)seg * C + k) * r;
      const bool ok = k < C;
      if (r == kRankPad && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {   // full rank: the 32-byte row in two vector loads
        uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
        if (ok) { q0 = reinterpret_cast<const uint4*>(src)[0]; q1 = reinterpret_cast<const uint4*>(src)[1]; }
        const uint32_t w32[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int n = 0; n < kRankPad; ++n) wv[n] = static_cast<unsigned short>((w32[n >> 1] >> (16 * (n & 1))) & 0xFFFFu);
      } else {
#pragma unroll
        for (int n = 0; n < kRankPad; ++n) wv[n] = (ok && n < r) ? src[n] : (unsigned short)0;
      }
    };
    auto store_w = [&](int ch) {
      uint8_t* dst = sm + (ch % kDownStages) * kDownStageBytes + kDownXBytes + threadIdx.x * 2;
#pragma unroll
      for (int n = 0; n < kRankPad; ++n)
        if (n < r) *reinterpret_cast<unsigned short*>(dst + n * kDownStride) = wv[n];
    };

    for (int pre = 0; pre < kDownStages - 1; ++pre) {
      if (pre < total_chunks) {
        issue_x(pre);
        if (kWisCR) { load_w(pre); store_w(pre); }
      }
      cp_async_commit();
    }
    for (int ch = 0; ch < total_chunks; ++ch) {
      const int nxt = ch + kDownStages - 1;
      if (nxt < total_chunks) {
        issue_x(nxt);
        if (kWisCR) load_w(nxt);   // lands in registers while this chunk is multiplied
      }
      cp_async_commit();
      cp_async_wait<kDownStages - 1>();
      __syncthreads();
      const uint32_t tile = sbase + (ch % kDownStages) * kDownStageBytes;
      const uint32_t wtile = tile + kDownXBytes;
#pragma unroll
      for (int kk = 0; kk < kDownBK / 16; ++kk) {
        uint32_t a[4], b[4];
        ldmatrix_x4(tile + (warp * 16 + (lane & 15)) * kDownStride + (kk * 16 + (lane >> 4) * 8) * 2, a);
        // W^T tile rows = rank index n, columns = k: matrices (n0-7,k0-7) (n0-7,k8-15) (n8-15,k0-7) (n8-15,k8-15)
        ldmatrix_x4(wtile + ((lane & 7) + ((lane >> 4) << 3)) * kDownStride + (kk * 16 + ((lane >> 3) & 1) * 8) * 2, b);
        mma_bf16(acc[0], a, b[0], b[1]);
        mma_bf16(acc[1], a, b[2], b[3]);
      }
      if (kWisCR && nxt < total_chunks) store_w(nxt);  // stage (ch-1)%3: every warp finished reading it before this iteration's barrier
      __syncthreads();
    }
    cp_async_wait<0>();
    // store: thread holds rows g and g+8, columns nt*8 + 2*(lane%4) + {0,1}
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = warp * 16 + (lane >> 2) + half * 8;
      if (row < s.rows) {
        const int64_t o = (int64_t)(s.row0 + row) * kRankPad;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = nt * 8 + (lane & 3) * 2;
          const float v0 = acc[nt][half * 2], v1 = acc[nt][half * 2 + 1];
          if (out_plain) *reinterpret_cast<uint32_t*>(out_plain + o + col) = dev::pack_bf16(v0, v1);
          if (out_scaled) *reinterpret_cast<uint32_t*>(out_scaled + o + col) = dev::pack_bf16(v0 * scale, v1 * scale);
        }
      }
    }
    __syncthreads();  // the next item's prologue rewrites stages this item may still be reading
  }
}

// ------------------------------------------------------------------------------------------------
// The same projection with the tiles brought in by TMA (weights given as [r, C], C a multiple of 64): one producer lane keeps
// a ring of [64 rows x 128 columns] activation tiles and [16 x 128] weight slices full across slice and item boundaries, the
// four MMA warps meet it only through mbarriers (no CTA-wide barrier anywhere), and nobody computes addresses or
// predicates per 16 bytes.  Tiles are two 128B-swizzled boxes of 64 columns each; rows past the matrix and columns past C arrive
// as zeros, rows past a ragged segment are computed and not stored, and rank rows >= r (another expert's, or zeros) are masked
// at the store.
// ------------------------------------------------------------------------------------------------
constexpr int kDtStages = 4;
constexpr int kDtXHalf = kDownRows * 128, kDtWHalf = kRankPad * 128;            // 8192, 2048 bytes
constexpr int kDtStageBytes = 2 * kDtXHalf + 2 * kDtWHalf;                        // 20480
constexpr int kDtSmemBytes = kDtStages * kDtStageBytes + 2 * kDtStages * 8 + 16 + 1024;

__global__ void __launch_bounds__(160) lora_down_tma_kernel(const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
                                                            const __grid_constant__ CUtensorMap tm_w, int nseg, float scale,
                                                            const int4* __restrict__ tiles, __nv_bfloat16* __restrict__ out_plain,
                                                            __nv_bfloat16* __restrict__ out_scaled, int64_t m_total, int C, int r,
                                                            int dense_rows) {
  extern __shared__ uint8_t sm_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sm_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = dev::smem_u32(sm);
  const uint32_t bars = sbase + kDtStages * kDtStageBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kDtStages * kDtStageBytes + 2 * kDtStages * 8);
  auto full = [&](int i) { return bars + 8u * i; };
  auto empty = [&](int i) { return bars + 8u * (kDtStages + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kDtStages; ++i) { dev::mbar_init(full(i), 1); dev::mbar_init(empty(i), 4); }
    *abort_flag = 0;
    dev::fence_barrier_init();
    dev::fence_proxy_async_smem();
  }
  __syncthreads();
  const int chunks = (C + kDownBK - 1) / kDownBK, total_chunks = nseg * chunks;
  const int total_items = tiles ? tiles[0].x * (tiles[0].y / kDownRows) : (int)gridDim.x * ((dense_rows + kDownRows - 1) / kDownRows);
  int st = 0, ph = 0;
  if (warp == 4) {
    if (lane == 0) {
      for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        const Seg s = down_segment(tiles, m_total, item, dense_rows);
        if (s.rows <= 0) continue;
        for (int ch = 0; ch < total_chunks; ++ch) {
          const int seg = ch / chunks, c0 = (ch - seg * chunks) * kDownBK;
          if (!dev::mbar_wait(empty(st), ph ^ 1, abort_flag, nullptr, 0)) return;
          dev::mbar_arrive_expect_tx(full(st), kDtStageBytes);
          const uint32_t dst = sbase + st * kDtStageBytes;
          const CUtensorMap* xm = seg ? &tm_x1 : &tm_x0;
          dev::tma_load_2d(dst, xm, full(st), c0, s.row0);
          dev::tma_load_2d(dst + kDtXHalf, xm, full(st), c0 + 64, s.row0);
          dev::tma_load_2d(dst + 2 * kDtXHalf, &tm_w, full(st), seg * C + c0, s.expert * r);
          dev::tma_load_2d(dst + 2 * kDtXHalf + kDtWHalf, &tm_w, full(st), seg * C + c0 + 64, s.expert * r);
          if (++st == kDtStages) { st = 0; ph ^= 1; }
        }
      }
    }
    return;
  }
  // ---- MMA warps: 16 rows each -------------------------------------------------------------------
  const int arow = warp * 16 + (lane & 15);                       // this lane's row of the activation tile (ldmatrix address)
  const uint32_t a_off = arow * 128u, a_sw = static_cast<uint32_t>(arow & 7), a_k = static_cast<uint32_t>(lane >> 4);
  const int wrow = (lane & 7) + ((lane >> 4) << 3);               // rank row of the weight slice
  const uint32_t w_off = wrow * 128u, w_sw = static_cast<uint32_t>(wrow & 7), w_k = static_cast<uint32_t>((lane >> 3) & 1);
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const Seg s = down_segment(tiles, m_total, item, dense_rows);
    if (s.rows <= 0) continue;
    float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    for (int ch = 0; ch < total_chunks; ++ch) {
      if (!dev::mbar_wait(full(st), ph, abort_flag, nullptr, 0)) return;
      const uint32_t xt = sbase + st * kDtStageBytes, wt = xt + 2 * kDtXHalf;
#pragma unroll
      for (int kk = 0; kk < kDownBK / 16; ++kk) {
        const uint32_t h = kk >> 2, j = 2u * (kk & 3);             // 64-column half, first 16-byte chunk of this k-slice in it
        uint32_t a[4], b[4];
        ldmatrix_x4(xt + h * kDtXHalf + a_off + (((j + a_k) ^ a_sw) << 4), a);
        ldmatrix_x4(wt + h * kDtWHalf + w_off + (((j + w_k) ^ w_sw) << 4), b);
        mma_bf16(acc[0], a, b[0], b[1]);
        mma_bf16(acc[1], a, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(empty(st));
      if (++st == kDtStages) { st = 0; ph ^= 1; }
    }
    // store: thread holds rows g and g+8, columns nt*8 + 2*(lane%4) + {0,1}; rank columns >= r are zero by definition
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = warp * 16 + (lane >> 2) + half * 8;
      if (row < s.rows) {
        const int64_t o = (int64_t)(s.row0 + row) * kRankPad;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = nt * 8 + (lane & 3) * 2;
          const float v0 = col < r ? acc[nt][half * 2] : 0.f, v1 = col + 1 < r ? acc[nt][half * 2 + 1] : 0.f;
          if (out_plain) *reinterpret_cast<uint32_t*>(out_plain + o + col) = dev::pack_bf16(v0, v1);
          if (out_scaled) *reinterpret_cast<uint32_t*>(out_scaled + o + col) = dev::pack_bf16(v0 * scale, v1 * scale);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Factor gradient: G[16, 128-column chunk] = S[rows,16]^T . T[rows, chunk] over one row segment.
// CTA = 4 warps x 32 columns; rows stream in steps of 64 through a 4-stage cp.async ring.
//   kPartial = true : dense path, segment = one split of M, fp32 partial to the workspace
//   kPartial = false: grouped path, segment = one expert, scaled bf16 straight to the output
// ------------------------------------------------------------------------------------------------
constexpr int kWgCols = 128, kWgRows = 64, kWgStages = 4, kWgTStride = kWgCols * 2 + 16, kWgSStride = 48;
constexpr int kWgStageBytes = kWgRows * kWgTStride + kWgRows * kWgSStride;

template <bool kPartial>
__global__ void __launch_bounds__(128) lora_wgrad_kernel(const __nv_bfloat16* __restrict__ s, const __nv_bfloat16* __restrict__ t, float scale,
                                                         const int32_t* __restrict__ offsets, int64_t m_total, int rows_per_split,
                                                         int C, int r, float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                         int transpose_out, int64_t out_col_offset, int64_t out_cols_total,
                                                         const int32_t* __restrict__ first_row) {
  extern __shared__ __align__(16) uint8_t sm[];
  const uint32_t sbase = dev::smem_u32(sm);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x, segi = blockIdx.y;
  const int c0 = chunk * kWgCols;
  int64_t row0, rows;
  if (kPartial) {
    row0 = (int64_t)segi * rows_per_split;
    rows = m_total - row0 < rows_per_split ? m_total - row0 : rows_per_split;
    if (rows < 0) rows = 0;
  } else {
    // offsets that overrun the operand (a receive buffer that was too small) are clamped to it
    row0 = segi > 0 ? offsets[segi - 1] : (first_row ? *first_row : 0);
    int64_t end = offsets[segi];
    if (row0 > m_total) row0 = m_total;
    if (end > m_total) end = m_total;
    rows = end > row0 ? end - row0 : 0;
  }
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int steps = (int)((rows + kWgRows - 1) / kWgRows);
  auto issue = [&](int st) {
    const uint32_t dst_t = sbase + (st % kWgStages) * kWgStageBytes;
    const uint32_t dst_s = dst_t + kWgRows * kWgTStride;
    const int64_t base = row0 + (int64_t)st * kWgRows;
    const int live = (int)(rows - (int64_t)st * kWgRows < kWgRows ? rows - (int64_t)st * kWgRows : kWgRows);
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // T tile: 64 rows x 16 vectors
      const int v = threadIdx.x + i * 128;
      const int row = v >> 4, vec = v & 15;
      const bool ok = row < live && c0 + vec * 8 < C;
      cp_async16(dst_t + row * kWgTStride + vec * 16, t + (base + (ok ? row : 0)) * C + c0 + (ok ? vec * 8 : 0), ok);
    }
    {  // S tile: 64 rows x 2 vectors
      const int row = threadIdx.x >> 1, vec = threadIdx.x & 1;
      const bool ok = row < live;
      cp_async16(dst_s + row * kWgSStride + vec * 16, s + (base + (ok ? row : 0)) * kRankPad + vec * 8, ok);
    }
  };
  for (int pre = 0; pre < kWgStages - 1; ++pre) {
    if (pre < steps) issue(pre);
    cp_async_commit();
  }
  for (int st = 0; st < steps; ++st) {
    if (st + kWgStages - 1 < steps) issue(st + kWgStages - 1);
    cp_async_commit();
    cp_async_wait<kWgStages - 1>();
    __syncthreads();
    const uint32_t tt = sbase + (st % kWgStages) * kWgStageBytes;
    const uint32_t ss = tt + kWgRows * kWgTStride;
#pragma unroll
    for (int kk = 0; kk < kWgRows / 16; ++kk) {
      uint32_t a[4];  // S^T fragment: rows = rank index, k = token row
      ldmatrix_x4_trans(ss + (kk * 16 + (lane >> 4) * 8 + (lane & 7)) * kWgSStride + ((lane >> 3) & 1) * 16, a);
#pragma unroll
      for (int np = 0; np < 2; ++np) {  // two pairs of 8-column tiles
        uint32_t b[4];
        ldmatrix_x4_trans(tt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kWgTStride + (warp * 32 + np * 16 + (lane >> 4) * 8) * 2, b);
        mma_bf16(acc[np * 2], a, b[0], b[1]);
        mma_bf16(acc[np * 2 + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  // acc[nt]: rank rows g, g+8; columns c0 + warp*32 + nt*8 + 2*(lane%4) + {0,1}
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = (lane >> 2) + half * 8;
      const int col = c0 + warp * 32 + nt * 8 + (lane & 3) * 2;
      if (col >= C) continue;
      const float v0 = acc[nt][half * 2], v1 = acc[nt][half * 2 + 1];
      if (kPartial) {
        float* p = partial + ((int64_t)segi * kRankPad + i) * C + col;
        p[0] = v0; p[1] = v1;
      } else if (i < r) {
        if (transpose_out) {
          __nv_bfloat16* o = out + ((int64_t)segi * out_cols_total + out_col_offset + col) * r + i;
          o[0] = __float2bfloat16_rn(v0 * scale);
          o[r] = __float2bfloat16_rn(v1 * scale);
        } else {
          __nv_bfloat16* o = out + ((int64_t)segi * r + i) * out_cols_total + out_col_offset + col;
          o[0] = __float2bfloat16_rn(v0 * scale);
          o[1] = __float2bfloat16_rn(v1 * scale);
        }
      }
    }
  }
}

// The dense factor gradient with the tiles brought in by TMA: a split is a whole number of 64-row steps (only the last one can
// run past the matrix, and rows past it arrive as zeros in S and T alike, so they add nothing), one producer lane keeps a ring of
// [64 x 128] T tiles (two 128B-swizzled boxes) and [64 x 16] S tiles (32B swizzle) full, and the four MMA warps meet it only
// through mbarriers.  Same fragments, same order and same partials as lora_wgrad_kernel<true>.
constexpr int kWtStages = 4;
constexpr int kWtTHalf = kWgRows * 128, kWtS = kWgRows * 32;                    // 8192, 2048 bytes
constexpr int kWtStageBytes = 2 * kWtTHalf + kWtS;                                // 18432
constexpr int kWtSmemBytes = kWtStages * kWtStageBytes + 2 * kWtStages * 8 + 16 + 1024;

__global__ void __launch_bounds__(160) lora_wgrad_tma_kernel(const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_t,
                                                             int64_t m_total, int rows_per_split, int C, float* __restrict__ partial) {
  extern __shared__ uint8_t sm_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sm_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = dev::smem_u32(sm);
  const uint32_t bars = sbase + kWtStages * kWtStageBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kWtStages * kWtStageBytes + 2 * kWtStages * 8);
  auto full = [&](int i) { return bars + 8u * i; };
  auto empty = [&](int i) { return bars + 8u * (kWtStages + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kWtStages; ++i) { dev::mbar_init(full(i), 1); dev::mbar_init(empty(i), 4); }
    *abort_flag = 0;
    dev::fence_barrier_init();
    dev::fence_proxy_async_smem();
  }
  __syncthreads();
  const int chunk = blockIdx.x, segi = blockIdx.y;
  const int c0 = chunk * kWgCols;
  const int64_t row0 = (int64_t)segi * rows_per_split;
  int64_t rows = m_total - row0 < rows_per_split ? m_total - row0 : rows_per_split;
  if (rows < 0) rows = 0;
  const int steps = (int)((rows + kWgRows - 1) / kWgRows);
  if (warp == 4) {
    if (lane == 0) {
      int st = 0, ph = 0;
      for (int i = 0; i < steps; ++i) {
        if (!dev::mbar_wait(empty(st), ph ^ 1, abort_flag, nullptr, 0)) return;
        dev::mbar_arrive_expect_tx(full(st), kWtStageBytes);
        const uint32_t dst = sbase + st * kWtStageBytes;
        const int y = (int)(row0 + (int64_t)i * kWgRows);
        dev::tma_load_2d(dst, &tm_t, full(st), c0, y);
        dev::tma_load_2d(dst + kWtTHalf, &tm_t, full(st), c0 + 64, y);
        dev::tma_load_2d(dst + 2 * kWtTHalf, &tm_s, full(st), 0, y);
        if (++st == kWtStages) { st = 0; ph ^= 1; }
      }
    }
    return;
  }
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  int st = 0, ph = 0;
  for (int i = 0; i < steps; ++i) {
    if (!dev::mbar_wait(full(st), ph, abort_flag, nullptr, 0)) return;
    const uint32_t tt = sbase + st * kWtStageBytes, ss = tt + 2 * kWtTHalf;
#pragma unroll
    for (int kk = 0; kk < kWgRows / 16; ++kk) {
      uint32_t a[4];  // S^T fragment: rows = rank index, k = token row
      const uint32_t srow = kk * 16 + (lane >> 4) * 8 + (lane & 7), sch = (lane >> 3) & 1;
      ldmatrix_x4_trans(ss + srow * 32u + ((sch ^ ((srow >> 2) & 1u)) << 4), a);
      const uint32_t trow = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int np = 0; np < 2; ++np) {  // two pairs of 8-column tiles
        uint32_t b[4];
        const uint32_t idx = warp * 4 + np * 2 + (lane >> 4);         // 16-byte chunk of the 128-column row
        ldmatrix_x4_trans(tt + (idx >> 3) * kWtTHalf + trow * 128u + (((idx & 7u) ^ (trow & 7u)) << 4), b);
        mma_bf16(acc[np * 2], a, b[0], b[1]);
        mma_bf16(acc[np * 2 + 1], a, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) dev::mbar_arrive(empty(st));
    if (++st == kWtStages) { st = 0; ph ^= 1; }
  }
  // acc[nt]: rank rows g, g+8; columns c0 + warp*32 + nt*8 + 2*(lane%4) + {0,1}
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = (lane >> 2) + half * 8;
      const int col = c0 + warp * 32 + nt * 8 + (lane & 3) * 2;
      if (col >= C) continue;
      float* p = partial + ((int64_t)segi * kRankPad + i) * C + col;
      p[0] = acc[nt][half * 2];
      p[1] = acc[nt][half * 2 + 1];
    }
  }
}

// Sum the per-split partials in split order (deterministic), scale, round, store.
__global__ void __launch_bounds__(64) lora_wgrad_reduce_kernel(const float* __restrict__ partial, int splits, int C, int r, float scale,
                                                                __nv_bfloat16* __restrict__ out, int transpose_out) {
  const int64_t n = (int64_t)r * C;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx / C), c = (int)(idx - (int64_t)i * C);
    float sum = 0.f;
    int sp = 0;
    for (; sp + 8 <= splits; sp += 8) {   // eight loads in flight, summed in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = partial[((int64_t)(sp + u) * kRankPad + i) * C + c];
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += v[u];
    }
    for (; sp < splits; ++sp) sum += partial[((int64_t)sp * kRankPad + i) * C + c];
    const __nv_bfloat16 v = __float2bfloat16_rn(sum * scale);
    if (transpose_out) out[(int64_t)c * r + i] = v;
    else out[idx] = v;
  }
}

// ------------------------------------------------------------------------------------------------
// Up-projection from the rank: Y[row, n] = sum_j P[row, j] * W_e[n, j]  (j < r <= 16), one expert per
// row segment.  Bound by writing Y; used by the un-fused operator surface (the fused path folds this
// product into the quantized GEMM as one extra MMA step).
// ------------------------------------------------------------------------------------------------
template <bool kWisNR>
__global__ void __launch_bounds__(128) lora_up_kernel(const __nv_bfloat16* __restrict__ p, int ldp, const __nv_bfloat16* __restrict__ w,
                                                      const int32_t* __restrict__ offsets_full, int num_experts,
                                                      __nv_bfloat16* __restrict__ y, int64_t rows, int N, int r) {
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    // expert of this row: first e with offsets[e] > row (binary search; E is small)
    int lo = 0, hi = num_experts - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (offsets_full[mid] > row) hi = mid; else lo = mid + 1;
    }
    const __nv_bfloat16* we = w + (int64_t)lo * N * r;
    float pv[kRankPad];
#pragma unroll
    for (int j = 0; j < kRankPad; ++j) pv[j] = j < r ? __bfloat162float(p[row * ldp + j]) : 0.f;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < kRankPad; ++j)
        if (j < r) acc = fmaf(pv[j], __bfloat162float(kWisNR ? we[(int64_t)n * r + j] : we[(int64_t)j * N + n]), acc);
      y[row * N + n] = __float2bfloat16_rn(acc);
    }
  }
}

inline int wgrad_splits(int64_t M, int64_t C) {
  const int chunks = (int)((C + kWgCols - 1) / kWgCols);
  // One wave: two CTAs are resident per SM, and chunks * splits never exceeds that, so no CTA waits for a slot and
  // every CTA streams a long row range (measured: 4.1 / 5.0 TB/s at C = 2048 / 4096 against 3.7 / 4.8 with two waves).
  int splits = 2 * sm_count() / chunks;
  const int64_t max_splits = (M + kWgRows - 1) / kWgRows;
  if (splits > max_splits) splits = (int)max_splits;
  if (splits < 1) splits = 1;
  return splits;
}

}  // namespace lora
}  // namespace b2g

using namespace b2g;

static int lora_down_launch(const void* x, const void* x1, const void* w, int w_is_cr, float scale, const int32_t* tiles, void* out_plain,
                            void* out_scaled, int64_t M, int64_t C, int r, int num_experts, void* stream, const char* what) {
  B2G_REQUIRE(r >= 1 && r <= lora::kRankPad, "%s: rank %d outside 1..16", what, r);
  B2G_REQUIRE(C > 0 && C % 8 == 0, "%s: reduction width %lld must be a multiple of 8", what, (long long)C);
  B2G_REQUIRE(M >= 0 && M < (1ll << 31), "%s: bad row count", what);
  if (M == 0) return 0;
  B2G_REQUIRE(x && w && (out_plain || out_scaled), "%s: null pointer", what);
  B2G_REQUIRE(aligned16(x) && (!x1 || aligned16(x1)), "%s: activations must be 16-byte aligned", what);
  // [r, C] rows are streamed with 16-byte cp.async (C % 8 == 0 keeps every row on a 16-byte boundary once the base is);
  // [C, r] rows are read with scalar loads, with a checked vector fast path
  B2G_REQUIRE(w_is_cr || aligned16(w), "%s: a weight given as [r, C] must be 16-byte aligned", what);
  const size_t smem = (size_t)lora::kDownStages * lora::kDownStageBytes;
  int grid = sm_count() * 2;       // two resident CTAs per SM
  int dense_rows = 0;
  if (!tiles) {
    const int64_t slices = (M + lora::kDownRows - 1) / lora::kDownRows;
    if (slices < grid) grid = (int)slices;
    dense_rows = (int)(((M + grid - 1) / grid + 15) / 16 * 16);   // whole 16-row MMA blocks
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* xb = static_cast<const __nv_bfloat16*>(x);
  auto* x1b = static_cast<const __nv_bfloat16*>(x1);
  auto* wb = static_cast<const __nv_bfloat16*>(w);
  auto* op = static_cast<__nv_bfloat16*>(out_plain);
  auto* os = static_cast<__nv_bfloat16*>(out_scaled);
  auto* tl = reinterpret_cast<const int4*>(tiles);
  if (!w_is_cr && C % 64 == 0) {
    // TMA-fed form.  Tensor maps: activations [M, C], weights [experts * r, nseg * C].
    const int nseg = x1 ? 2 : 1;
    CUtensorMap tm_x0, tm_x1, tm_w;
    int rc;
    if ((rc = make_tmap_2d(&tm_x0, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)C, (uint64_t)M, (uint64_t)C * 2, 64, lora::kDownRows,
                           CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    tm_x1 = tm_x0;
    if (x1 && (rc = make_tmap_2d(&tm_x1, x1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)C, (uint64_t)M, (uint64_t)C * 2, 64,
                                 lora::kDownRows, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap_2d(&tm_w, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)nseg * C, (uint64_t)num_experts * r,
                           (uint64_t)nseg * C * 2, 64, lora::kRankPad, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    B2G_KERNEL_SMEM(lora::lora_down_tma_kernel, lora::kDtSmemBytes);
    lora::lora_down_tma_kernel<<<grid, 160, lora::kDtSmemBytes, s>>>(tm_x0, tm_x1, tm_w, nseg, scale, tl, op, os, M, (int)C, r, dense_rows);
  } else if (w_is_cr) {
    B2G_KERNEL_SMEM(lora::lora_down_kernel<true>, smem);
    lora::lora_down_kernel<true><<<grid, 128, smem, s>>>(xb, x1b, wb, scale, tl, op, os, M, (int)C, r, dense_rows);
  } else {
    B2G_KERNEL_SMEM(lora::lora_down_kernel<false>, smem);
    lora::lora_down_kernel<false><<<grid, 128, smem, s>>>(xb, x1b, wb, scale, tl, op, os, M, (int)C, r, dense_rows);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_lora_down(const void* x, const void* w, int w_is_cr, float scale, void* out_plain, void* out_scaled, int64_t M,
                             int64_t C, int r, void* stream) {
  return lora_down_launch(x, nullptr, w, w_is_cr, scale, nullptr, out_plain, out_scaled, M, C, r, 1, stream, "lora_down");
}

extern "C" int b2g_grouped_lora_down(const void* x, const void* x1, const void* w, int w_is_cr, float scale, const int32_t* tiles,
                                     void* out_plain, void* out_scaled, int64_t R, int64_t C, int r, int num_experts, void* stream) {
  B2G_REQUIRE(tiles != nullptr && num_experts >= 1, "grouped_lora_down: tile table missing");
  return lora_down_launch(x, x1, w, w_is_cr, scale, tiles, out_plain, out_scaled, R, C, r, num_experts, stream, "grouped_lora_down");
}

extern "C" int64_t b2g_lora_wgrad_workspace_bytes(int64_t M, int64_t C) {
  if (M <= 0 || C <= 0) return 16;
  return (int64_t)lora::wgrad_splits(M, C) * lora::kRankPad * C * (int64_t)sizeof(float);
}

extern "C" int b2g_lora_wgrad(const void* s, const void* t, float scale, void* out, int transpose_out, void* workspace,
                              int64_t workspace_bytes, int64_t M, int64_t C, int r, void* stream) {
  B2G_REQUIRE(r >= 1 && r <= lora::kRankPad, "lora_wgrad: rank %d outside 1..16", r);
  B2G_REQUIRE(C > 0 && C % 8 == 0 && M > 0 && M < (1ll << 31), "lora_wgrad: bad shape M=%lld C=%lld", (long long)M, (long long)C);
  B2G_REQUIRE(s && t && out && workspace, "lora_wgrad: null pointer");
  B2G_REQUIRE(aligned16(s) && aligned16(t) && aligned16(workspace), "lora_wgrad: operands must be 16-byte aligned");
  B2G_REQUIRE(workspace_bytes >= b2g_lora_wgrad_workspace_bytes(M, C), "lora_wgrad: workspace of %lld bytes is smaller than %lld",
              (long long)workspace_bytes, (long long)b2g_lora_wgrad_workspace_bytes(M, C));
  const int splits = lora::wgrad_splits(M, C);
  int rows_per_split = (int)((M + splits - 1) / splits);
  rows_per_split = (rows_per_split + lora::kWgRows - 1) / lora::kWgRows * lora::kWgRows;
  const int chunks = (int)((C + lora::kWgCols - 1) / lora::kWgCols);
  const size_t smem = (size_t)lora::kWgStages * lora::kWgStageBytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B2G_KERNEL_MAX_SHARED(lora::lora_wgrad_reduce_kernel);
  {
    // TMA-fed form.  Tensor maps: S [M, 16] (32-byte rows), T [M, C].
    (void)smem;
    CUtensorMap tm_s, tm_t;
    int rc;
    if ((rc = make_tmap_2d(&tm_s, s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lora::kRankPad, (uint64_t)M, lora::kRankPad * 2, lora::kRankPad,
                           lora::kWgRows, CU_TENSOR_MAP_SWIZZLE_32B))) return rc;
    if ((rc = make_tmap_2d(&tm_t, t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)C, (uint64_t)M, (uint64_t)C * 2, 64, lora::kWgRows,
                           CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    B2G_KERNEL_SMEM(lora::lora_wgrad_tma_kernel, lora::kWtSmemBytes);
    lora::lora_wgrad_tma_kernel<<<dim3(chunks, splits), 160, lora::kWtSmemBytes, st>>>(tm_s, tm_t, M, rows_per_split, (int)C,
                                                                                       static_cast<float*>(workspace));
  }
  B2G_CUDA_OK(cudaGetLastError());
  const int64_t n = (int64_t)r * C;
  lora::lora_wgrad_reduce_kernel<<<(int)((n + 63) / 64), 64, 0, st>>>(static_cast<const float*>(workspace), splits, (int)C, r, scale,
                                                                       static_cast<__nv_bfloat16*>(out), transpose_out);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_grouped_lora_wgrad(const void* s, const void* t, float scale, const int32_t* offsets_full, const int32_t* first_row,
                                      void* out, int transpose_out, int64_t R, int64_t C, int r, int num_experts, int64_t out_col_offset,
                                      int64_t out_cols_total, void* stream) {
  B2G_REQUIRE(r >= 1 && r <= lora::kRankPad, "grouped_lora_wgrad: rank %d outside 1..16", r);
  B2G_REQUIRE(C > 0 && C % 8 == 0 && R >= 0, "grouped_lora_wgrad: bad shape");
  B2G_REQUIRE(num_experts >= 1 && num_experts <= 65535, "grouped_lora_wgrad: bad expert count %d", num_experts);
  B2G_REQUIRE(s && t && out && offsets_full, "grouped_lora_wgrad: null pointer");
  B2G_REQUIRE(aligned16(s) && aligned16(t), "grouped_lora_wgrad: operands must be 16-byte aligned");
  B2G_REQUIRE(out_col_offset >= 0 && out_col_offset + C <= out_cols_total, "grouped_lora_wgrad: output slice out of range");
  const int chunks = (int)((C + lora::kWgCols - 1) / lora::kWgCols);
  const size_t smem = (size_t)lora::kWgStages * lora::kWgStageBytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B2G_KERNEL_SMEM(lora::lora_wgrad_kernel<false>, smem);
  lora::lora_wgrad_kernel<false><<<dim3(chunks, num_experts), 128, smem, st>>>(
      static_cast<const __nv_bfloat16*>(s), static_cast<const __nv_bfloat16*>(t), scale, offsets_full, R, 0, (int)C, r, nullptr,
      static_cast<__nv_bfloat16*>(out), transpose_out, out_col_offset, out_cols_total, first_row);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_grouped_lora_up(const void* p, int64_t ldp, const void* w, int w_is_nr, const int32_t* offsets_full, void* y,
                                   int64_t R, int64_t N, int r, int num_experts, void* stream) {
  B2G_REQUIRE(r >= 1 && r <= lora::kRankPad && ldp >= r, "grouped_lora_up: rank %d / row stride %lld invalid", r, (long long)ldp);
  B2G_REQUIRE(N > 0 && R >= 0 && num_experts >= 1, "grouped_lora_up: bad shape");
  if (R == 0) return 0;
  B2G_REQUIRE(p && w && y && offsets_full, "grouped_lora_up: null pointer");
  const int64_t cap = (int64_t)sm_count() * 16;
  const int grid = (int)(R < cap ? R : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (w_is_nr)
    lora::lora_up_kernel<true><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(p), (int)ldp, static_cast<const __nv_bfloat16*>(w),
                                                     offsets_full, num_experts, static_cast<__nv_bfloat16*>(y), R, (int)N, r);
  else
    lora::lora_up_kernel<false><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(p), (int)ldp, static_cast<const __nv_bfloat16*>(w),
                                                      offsets_full, num_experts, static_cast<__nv_bfloat16*>(y), R, (int)N, r);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Factor gradient for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or ask torch's allocator) at the point where the
// gradient is needed: code running inside another framework's memory plan, a plug-in that was handed
// only its input and output buffers, or a process whose memory pool is already fully committed.  For
// them the split partials live in the fixed array below instead of a caller-provided workspace.  The
// array is part of the library image: every GPU that loads the library holds these bytes until exit.
// ------------------------------------------------------------------------------------------------
namespace b2g {
namespace lora {
constexpr int64_t kStaticScratchBytes = 8ll << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_wgrad_scratch[kStaticScratchBytes];
}  // namespace lora
}  // namespace b2g

// In host code `g_wgrad_scratch` is only a handle for the symbol, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress, fetched once per device with that device current.
static int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  B2G_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    B2G_CUDA_OK(cudaGetSymbolAddress(&p, b2g::lora::g_wgrad_scratch));
    B2G_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return 0;
}

extern "C" int64_t b2g_lora_wgrad_static_max_bytes(void) { return b2g::lora::kStaticScratchBytes; }

extern "C" int b2g_lora_wgrad_static(const void* s, const void* t, float scale, void* out, int transpose_out, int64_t M, int64_t C,
                                     int r, void* stream) {
  B2G_REQUIRE(M > 0 && C > 0, "lora_wgrad_static: bad shape M=%lld C=%lld", (long long)M, (long long)C);
  const int64_t need = b2g_lora_wgrad_workspace_bytes(M, C);
  B2G_REQUIRE(need <= b2g::lora::kStaticScratchBytes,
              "lora_wgrad_static: M=%lld, C=%lld needs %lld bytes of scratch, the built-in array holds %lld; use b2g_lora_wgrad with "
              "a caller-provided workspace", (long long)M, (long long)C, (long long)need, (long long)b2g::lora::kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  // Every partial the reduction reads is written by the first kernel of this call, so nothing has to be cleared.
  return b2g_lora_wgrad(s, t, scale, out, transpose_out, scratch, b2g::lora::kStaticScratchBytes, M, C, r, stream);
}
