// Stand-alone GGUF dequantiser: packed payload -> logical bf16 weight (HBM-bound streaming kernel).
#include "b2g_formats.cuh"

namespace b2g {
int iq2xxs_grid(const uint2** out);
int iq2s_grid(const uint2** out);

// One thread decodes 8 consecutive values and writes one 16-byte vector.  Consecutive threads take
// consecutive 8-value chunks of a row, so stores are fully coalesced; the packed bytes (0.26-1.06
// bytes per value) come through L1/L2.
template <int QT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ payload, int64_t rows, int cols,
                                                      int64_t pitch, const uint2* __restrict__ grid,
                                                      uint4* __restrict__ out) {
  const int chunks_per_row = cols >> 3;
  const int64_t total = rows * chunks_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks_per_row;
    const int c = static_cast<int>(i - r * chunks_per_row);
    float v[8];
    fmt::Decode8<QT>::run(payload + r * pitch, c * 8, grid, v);
    uint4 o;
    o.x = dev::pack_bf16(v[0], v[1]);
    o.y = dev::pack_bf16(v[2], v[3]);
    o.z = dev::pack_bf16(v[4], v[5]);
    o.w = dev::pack_bf16(v[6], v[7]);
    out[i] = o;
  }
}
}  // namespace b2g

extern "C" int b2g_dequant(int qtype, const void* payload, int64_t rows, int64_t cols, void* out_bf16, void* stream) {
  using namespace b2g;
  B2G_REQUIRE(qtype == B2G_Q8_0 || qtype == B2G_Q4_K || qtype == B2G_IQ2_XXS || qtype == B2G_Q6_K || qtype == B2G_Q5_K || qtype == B2G_Q2_K || qtype == B2G_Q3_K || qtype == B2G_IQ2_S, "unsupported GGUF type id %d", qtype);
  B2G_REQUIRE(rows >= 0 && cols > 0 && cols % fmt::block_values(qtype) == 0,
              "cols=%lld is not a multiple of the %d-value block", (long long)cols, fmt::block_values(qtype));
  B2G_REQUIRE(cols < (1ll << 31), "cols too large");
  if (rows == 0) return 0;
  B2G_REQUIRE(payload && out_bf16, "null pointer");
  B2G_REQUIRE(aligned16(payload) && aligned16(out_bf16), "payload and output must be 16-byte aligned");
  const int64_t pitch = fmt::row_bytes(qtype, cols);
  const int64_t total = rows * (cols / 8);
  int64_t want = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint8_t* p = static_cast<const uint8_t*>(payload);
  uint4* o = static_cast<uint4*>(out_bf16);
  if (qtype == B2G_Q8_0) {
    dequant_kernel<B2G_Q8_0><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else if (qtype == B2G_Q4_K) {
    dequant_kernel<B2G_Q4_K><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else if (qtype == B2G_Q2_K) {
    B2G_REQUIRE(fmt::row_bytes(qtype, cols) % 4 == 0, "Q2_K rows must be 4-byte multiples");
    dequant_kernel<B2G_Q2_K><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else if (qtype == B2G_IQ2_S) {
    const uint2* grid = nullptr;
    int rc = iq2s_grid(&grid);
    if (rc) return rc;
    dequant_kernel<B2G_IQ2_S><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, grid, o);
  } else if (qtype == B2G_Q3_K) {
    dequant_kernel<B2G_Q3_K><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else if (qtype == B2G_Q5_K) {
    dequant_kernel<B2G_Q5_K><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else if (qtype == B2G_Q6_K) {
    dequant_kernel<B2G_Q6_K><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, nullptr, o);
  } else {
    const uint2* grid = nullptr;
    int rc = iq2xxs_grid(&grid);
    if (rc) return rc;
    dequant_kernel<B2G_IQ2_XXS><<<blocks, 256, 0, s>>>(p, rows, (int)cols, pitch, grid, o);
  }
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}
