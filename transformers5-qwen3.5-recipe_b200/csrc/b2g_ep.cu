// Expert-parallel row exchange over peer memory: the token permute and the inter-GPU transfer are one pass.
//
// Every rank maps the receive buffers of all ranks (NVLink peer pointers of a symmetric allocation).
//   scatter: for each routed row, sorted by global expert id on the SOURCE rank, copy the token's row straight
//            into the OWNER rank's receive buffer, at the slot that groups rows by (local expert, source rank).
//            One launch moves one EXPERT GROUP (a range of local expert indices, the same on every owner), so that
//            the experts of one group can compute while the next group's rows are still crossing NVLink.
//            With `perm` the source row is gathered from the token matrix on the fly (dispatch of activations);
//            without it rows are taken in order (dispatch of output gradients).
//   return : the inverse on the OWNER rank: each row of the grouped buffer goes back to its source rank, to the
//            position it has in that rank's sorted order (combine of expert outputs / of input gradients).
// Slots come from the all-gathered count matrix, so no split size ever visits the host.  Plain 16-byte peer
// stores only: no multicast, no waits inside the kernels (ranks synchronise between the two phases on the
// stream, outside these kernels).
//
// The two copy kernels are built to run BESIDE the quantized GEMM on the same SMs, so that an exchange of one
// token chunk on its own stream proceeds while the expert products of another chunk compute.  The GEMM's CTA
// (23 warps of 80 registers) takes six warps' worth of registers in three of the SM's four register files and
// five in the fourth, which leaves 1024 registers in each of the three: room for exactly one warp of 32
// registers per file.  Hence 128 threads (one warp per file), at most 32 registers, no shared memory, one CTA
// per SM, and the largest shared-memory partition requested so that the SM need not be re-partitioned (which
// it cannot be while a CTA is resident) when the GEMM moves in.
//
// A receive buffer that is too small is CONTAINED, not only reported: the plan kernel clamps every segment
// of the rows this rank receives to the buffer's capacity (and sets status 901), so that the grouped
// products that consume the plan never index past the buffer; the scatter kernel drops the rows that
// would land beyond it.
#include "b2g_common.cuh"

namespace b2g {
namespace ep {

// One warp copies one row, kVec 16-byte vectors per lane in flight: four in the small variant (its register budget of 32
// allows no more), eight in the wide one.
template <int kVec>
__device__ __forceinline__ void copy_row(const uint4* __restrict__ in, uint4* __restrict__ out, int vec_per_row, int lane) {
  for (int v0 = lane; v0 < vec_per_row; v0 += 32 * kVec) {
    uint4 buf[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (v0 + 32 * i < vec_per_row) buf[i] = __ldcs(in + v0 + 32 * i);
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (v0 + 32 * i < vec_per_row) out[v0 + 32 * i] = buf[i];
  }
}

// Two shapes of each copy kernel:
//   small: 128 threads, 32 registers, four vectors in flight per lane: fits beside the GEMM's CTA on the same SM;
//   wide : 1024 threads, 64 registers, eight vectors in flight per lane: fills an SM by itself.  Launched as clusters of two
//          CTAs, which the hardware places on the two SMs of one TPC, on a few TPCs that the GEMM (itself launched on CTA pairs
//          and told to leave that many SMs free) does not use: the exchange then shares no SM with the expert products.
struct Small { static constexpr int kThreads = 128, kMinBlocks = 16, kVec = 4; };
struct Wide { static constexpr int kThreads = 1024, kMinBlocks = 1, kVec = 8; };

// Scatter of the rows whose LOCAL expert index (global id modulo experts_per_rank) lies in [group_lo, group_hi): one expert group
// of every owner.  Rows are sorted by global expert id, so the group is one contiguous range of sorted positions per owner;
// the owners are visited one after the other, starting with the rank after this one, so that the ranks of a job do not all
// store to the same GPU at the same time (one NVLink port would take everything while the others idle).
template <typename Shape>
__global__ void __launch_bounds__(Shape::kThreads, Shape::kMinBlocks) scatter_rows_kernel(const uint4* __restrict__ src, const int64_t* __restrict__ perm, int top_k,
                                                               const int64_t* __restrict__ sorted_expert, const int32_t* __restrict__ my_start,
                                                               const int32_t* __restrict__ dest_base, const unsigned long long* __restrict__ peers,
                                                               int experts_per_rank, int world, int rank, int group_lo, int group_hi, int64_t R,
                                                               int vec_per_row, int64_t capacity, int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int step = 1; step <= world; ++step) {
    const int owner = (rank + step) % world;
    const int e_first = owner * experts_per_rank + group_lo, e_end = owner * experts_per_rank + group_hi;
    const int64_t s_begin = my_start[e_first];
    const int64_t s_end = e_end < world * experts_per_rank ? static_cast<int64_t>(my_start[e_end]) : R;
    uint4* const base = reinterpret_cast<uint4*>(peers[owner]);
    for (int64_t s = s_begin + warp; s < s_end; s += nwarps) {
      const int e = static_cast<int>(sorted_expert[s]);
      const int64_t slot = static_cast<int64_t>(dest_base[e]) + (s - my_start[e]);
      if (slot >= capacity) {
        if (lane == 0 && status) atomicCAS(status, 0, 901);   // receive buffer too small: report, never write past it
        continue;
      }
      const int64_t from = perm ? perm[s] / top_k : s;
      copy_row<Shape::kVec>(src + from * vec_per_row, base + slot * vec_per_row, vec_per_row, lane);
    }
  }
}

// The inverse on the owner: the rows of the blocks [block_lo, block_hi) (block b = local expert b / world, source rank b % world;
// an expert group is a contiguous range of blocks and of rows) go back to their sources.
template <typename Shape>
__global__ void __launch_bounds__(Shape::kThreads, Shape::kMinBlocks) return_rows_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ blk_start,
                                                              const int32_t* __restrict__ src_pos, const unsigned long long* __restrict__ peers,
                                                              int world, int block_lo, int block_hi, int vec_per_row, int64_t capacity) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t first = blk_start[block_lo];
  const int64_t total = blk_start[block_hi];
  const int64_t live = total < capacity ? total : capacity;
  for (int64_t j = first + warp; j < live; j += nwarps) {
    // block (local expert, source rank) that holds row j: last b in the range with blk_start[b] <= j
    int lo = block_lo, hi = block_hi - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (blk_start[mid] <= j) lo = mid; else hi = mid - 1;
    }
    const int64_t pos = static_cast<int64_t>(src_pos[lo]) + (j - blk_start[lo]);
    copy_row<Shape::kVec>(rows + j * vec_per_row, reinterpret_cast<uint4*>(peers[lo % world]) + pos * vec_per_row, vec_per_row, lane);
  }
}


// Slots of one rank from the all-gathered count matrix counts[G][E] (row g = histogram of rank g's routed rows over
// the global experts), one CTA, a few thousand integer operations:
//   my_start[e]   first position of expert e in THIS rank's sorted order
//   dest_base[e]  slot at e's owner where this rank's rows of e start (owner's earlier experts, then earlier sources)
//   blk_start[b]  owner side, b = local expert * G + source rank: first row of the block; blk_start[E_l*G] = rows held
//   src_pos[b]    position of that block's first row in the source rank's sorted order
//   local_sizes / local_offsets: rows per local expert and their cumulative ends
constexpr int kPlanMaxExperts = 2048, kPlanMaxRanks = 64;

__global__ void __launch_bounds__(256) peer_plan_kernel(const int32_t* __restrict__ counts, int64_t count_stride, int G, int E, int rank,
                                                        int32_t* __restrict__ my_start, int32_t* __restrict__ dest_base,
                                                        int32_t* __restrict__ blk_start, int32_t* __restrict__ src_pos,
                                                        int32_t* __restrict__ local_sizes, int32_t* __restrict__ local_offsets,
                                                        int64_t capacity, int* __restrict__ status) {
  __shared__ int32_t total[kPlanMaxExperts];
  const int per = E / G, lo = rank * per;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int32_t sum = 0, before = 0;
    for (int g = 0; g < G; ++g) {
      const int32_t c = counts[g * count_stride + e];
      sum += c;
      if (g < rank) before += c;
    }
    total[e] = sum;
    dest_base[e] = before;          // earlier sources; the owner's earlier experts are added below
  }
  __syncthreads();
  // one thread per owner rank: running sum of the totals of its experts
  for (int o = threadIdx.x; o < G; o += blockDim.x) {
    int32_t run = 0;
    for (int j = 0; j < per; ++j) {
      const int e = o * per + j;
      dest_base[e] += run;
      if (o == rank) {
        // what the grouped products may touch: segments clamped to the receive buffer
        const int64_t begin = run < capacity ? run : capacity;
        const int64_t end = (int64_t)run + total[e] < capacity ? (int64_t)run + total[e] : capacity;
        local_sizes[j] = static_cast<int32_t>(end - begin);
        local_offsets[j] = static_cast<int32_t>(end);
        if ((int64_t)run + total[e] > capacity && status) atomicCAS(status, 0, 901);
      }
      run += total[e];
    }
  }
  // one thread per source rank: where each of this rank's local experts starts in that source's sorted order
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    int32_t run = 0;
    for (int e = 0; e < E; ++e) {
      if (g == rank) my_start[e] = run;
      if (e >= lo && e < lo + per) src_pos[(e - lo) * G + g] = run;
      run += counts[g * count_stride + e];
    }
  }
  // blocks of the owner side in (local expert, source rank) order, clamped like the segments above
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int j = 0; j < per; ++j)
      for (int g = 0; g < G; ++g) {
        blk_start[j * G + g] = static_cast<int32_t>(run < capacity ? run : capacity);
        run += counts[g * count_stride + lo + j];
      }
    blk_start[per * G] = static_cast<int32_t>(run < capacity ? run : capacity);
  }
}

}  // namespace ep
}  // namespace b2g

using namespace b2g;

// `spread`: > 0 = the small kernel with that many CTAs per SM (1 to run beside the GEMM on the same SMs, more when nothing
// computes beside the exchange); < 0 = the wide kernel on -spread TPCs (cluster pairs) that the GEMM leaves free.

extern "C" int b2g_ep_scatter_rows(const void* src, const int64_t* perm, int top_k, const int64_t* sorted_expert, const int32_t* my_start,
                                   const int32_t* dest_base, const uint64_t* peer_ptrs, int experts_per_rank, int world, int rank,
                                   int group_lo, int group_hi, int64_t R, int H, int64_t capacity_rows, int spread, int* status,
                                   void* stream) {
  B2G_REQUIRE(H > 0 && H % 8 == 0, "ep_scatter_rows: row width %d must be a positive multiple of 8", H);
  B2G_REQUIRE(experts_per_rank >= 1 && capacity_rows >= 0 && R >= 0, "ep_scatter_rows: bad sizes");
  B2G_REQUIRE(world >= 1 && rank >= 0 && rank < world, "ep_scatter_rows: rank %d of %d", rank, world);
  B2G_REQUIRE(group_lo >= 0 && group_lo < group_hi && group_hi <= experts_per_rank, "ep_scatter_rows: expert group [%d, %d) outside 0..%d",
              group_lo, group_hi, experts_per_rank);
  B2G_REQUIRE(perm == nullptr || top_k >= 1, "ep_scatter_rows: top_k must be positive when rows are gathered");
  B2G_REQUIRE(spread != 0 && spread >= -64 && spread <= 16, "ep_scatter_rows: spread %d outside -64..-1, 1..16", spread);
  if (R == 0) return 0;
  B2G_REQUIRE(src && sorted_expert && my_start && dest_base && peer_ptrs && aligned16(src), "ep_scatter_rows: null or misaligned pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* peers = reinterpret_cast<const unsigned long long*>(peer_ptrs);
  if (spread > 0) {
    const int64_t want = (R + 3) / 4, cap = (int64_t)sm_count() * spread;
    B2G_KERNEL_MAX_SHARED(ep::scatter_rows_kernel<ep::Small>);
    ep::scatter_rows_kernel<ep::Small><<<(int)(want < cap ? want : cap), ep::Small::kThreads, 0, st>>>(
        static_cast<const uint4*>(src), perm, top_k, sorted_expert, my_start, dest_base, peers, experts_per_rank, world, rank, group_lo,
        group_hi, R, H / 8, capacity_rows, status);
    B2G_CUDA_OK(cudaGetLastError());
    return 0;
  }
  B2G_KERNEL_MAX_SHARED(ep::scatter_rows_kernel<ep::Wide>);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * -spread);
  cfg.blockDim = dim3(ep::Wide::kThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  B2G_CUDA_OK(cudaLaunchKernelEx(&cfg, ep::scatter_rows_kernel<ep::Wide>, static_cast<const uint4*>(src), perm, top_k, sorted_expert, my_start,
                                 dest_base, peers, experts_per_rank, world, rank, group_lo, group_hi, R, H / 8, capacity_rows, status));
  return 0;
}

extern "C" int b2g_ep_return_rows(const void* rows, const int32_t* blk_start, const int32_t* src_pos, const uint64_t* peer_ptrs, int world,
                                  int block_lo, int block_hi, int H, int64_t capacity_rows, int spread, void* stream) {
  B2G_REQUIRE(H > 0 && H % 8 == 0, "ep_return_rows: row width %d must be a positive multiple of 8", H);
  B2G_REQUIRE(world >= 1 && block_lo >= 0 && block_lo < block_hi && block_lo % world == 0 && block_hi % world == 0,
              "ep_return_rows: blocks [%d, %d) are not whole experts of %d ranks", block_lo, block_hi, world);
  B2G_REQUIRE(spread != 0 && spread >= -64 && spread <= 16, "ep_return_rows: spread %d outside -64..-1, 1..16", spread);
  if (capacity_rows == 0) return 0;
  B2G_REQUIRE(rows && blk_start && src_pos && peer_ptrs && aligned16(rows), "ep_return_rows: null or misaligned pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* peers = reinterpret_cast<const unsigned long long*>(peer_ptrs);
  if (spread > 0) {
    const int64_t want = (capacity_rows + 3) / 4, cap = (int64_t)sm_count() * spread;
    B2G_KERNEL_MAX_SHARED(ep::return_rows_kernel<ep::Small>);
    ep::return_rows_kernel<ep::Small><<<(int)(want < cap ? want : cap), ep::Small::kThreads, 0, st>>>(
        static_cast<const uint4*>(rows), blk_start, src_pos, peers, world, block_lo, block_hi, H / 8, capacity_rows);
    B2G_CUDA_OK(cudaGetLastError());
    return 0;
  }
  B2G_KERNEL_MAX_SHARED(ep::return_rows_kernel<ep::Wide>);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * -spread);
  cfg.blockDim = dim3(ep::Wide::kThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  B2G_CUDA_OK(cudaLaunchKernelEx(&cfg, ep::return_rows_kernel<ep::Wide>, static_cast<const uint4*>(rows), blk_start, src_pos, peers, world,
                                 block_lo, block_hi, H / 8, capacity_rows));
  return 0;
}

extern "C" int b2g_ep_peer_plan(const int32_t* counts, int64_t count_stride, int world, int num_experts, int rank, int32_t* my_start,
                                int32_t* dest_base, int32_t* blk_start, int32_t* src_pos, int32_t* local_sizes, int32_t* local_offsets,
                                int64_t capacity_rows, int* status, void* stream) {
  B2G_REQUIRE(world >= 1 && world <= ep::kPlanMaxRanks && num_experts >= world && num_experts <= ep::kPlanMaxExperts &&
                  num_experts % world == 0, "ep_peer_plan: %d experts over %d ranks is outside what one CTA plans (<= %d experts, <= %d ranks)",
              num_experts, world, ep::kPlanMaxExperts, ep::kPlanMaxRanks);
  B2G_REQUIRE(rank >= 0 && rank < world, "ep_peer_plan: rank %d of %d", rank, world);
  B2G_REQUIRE(counts && my_start && dest_base && blk_start && src_pos && local_sizes && local_offsets, "ep_peer_plan: null pointer");
  B2G_REQUIRE(count_stride >= num_experts && capacity_rows >= 0 && capacity_rows < (1ll << 31), "ep_peer_plan: bad count stride or capacity");
  B2G_KERNEL_MAX_SHARED(ep::peer_plan_kernel);
  ep::peer_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, count_stride, world, num_experts, rank, my_start, dest_base,
                                                                         blk_start, src_pos, local_sizes, local_offsets, capacity_rows, status);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}
