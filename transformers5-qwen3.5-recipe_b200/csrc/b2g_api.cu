// Library-wide host state of libb2g: error text, device properties, tensor-map encoding and the
// IQ2_XXS table upload.
#include "b2g_common.cuh"

#include <mutex>
#include <unordered_map>

#include <mutex>

namespace b2g {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoded tensor maps are kept per (base address, geometry): a training step presents the same tensors at the same addresses
// again and again (frozen payloads always, activations as often as the caching allocator returns the same block), and a map
// depends on nothing else.  The table is bounded; when it is full it is emptied and refills.
namespace {
struct TmapKey {
  const void* base; uint64_t inner, rows, pitch; uint32_t box_inner, box_rows; int dt, sw, dev;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && rows == o.rows && pitch == o.pitch && box_inner == o.box_inner && box_rows == o.box_rows &&
           dt == o.dt && sw == o.sw && dev == o.dev;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    for (uint64_t v : {k.inner, k.rows, k.pitch, (uint64_t)k.box_inner << 32 | k.box_rows, (uint64_t)k.dt << 40 | (uint64_t)k.sw << 20 | (uint64_t)k.dev})
      h = (h ^ v) * 0x100000001B3ull;
    return static_cast<size_t>(h ^ (h >> 29));
  }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
constexpr size_t kTmapCacheEntries = 8192;
}  // namespace

static int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner, uint64_t rows,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw);

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner,
                 uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw) {
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  const TmapKey key{base, inner, rows, pitch_bytes, box_inner, box_rows, (int)dt, (int)sw, dev};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) { *out = it->second; return 0; }
  }
  int rc = encode_tmap_2d(out, base, dt, elem_bytes, inner, rows, pitch_bytes, box_inner, box_rows, sw);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  if (g_tmaps.size() >= kTmapCacheEntries) g_tmaps.clear();
  g_tmaps.emplace(key, *out);
  return 0;
}

static int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner, uint64_t rows,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B2G_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (!aligned16(base)) return fail(B2G_E_ARG, "tensor base %p is not 16-byte aligned", base);
  if (pitch_bytes % 16) return fail(B2G_E_ARG, "row pitch %llu is not a multiple of 16 bytes", (unsigned long long)pitch_bytes);
  if ((uint64_t)box_inner * elem_bytes % 16) return fail(B2G_E_ARG, "box row of %u bytes is not a multiple of 16", box_inner * elem_bytes);
  if (rows == 0) rows = 1;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B2G_E_CUDA, "cuTensorMapEncodeTiled failed (%d): inner=%llu rows=%llu pitch=%llu box=%ux%u", (int)r,
                (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)pitch_bytes, box_inner, box_rows);
  return 0;
}

// IQ2_XXS magnitude table, one copy per device that uploaded it.
__device__ uint2 g_iq2xxs_grid[256];
static bool g_grid_ready[64] = {false};

int iq2xxs_grid(const uint2** out) {
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !g_grid_ready[dev])
    return fail(B2G_E_STATE, "IQ2_XXS grid not uploaded on device %d: call b2g_set_iq2xxs_grid first", dev);
  void* p = nullptr;
  B2G_CUDA_OK(cudaGetSymbolAddress(&p, g_iq2xxs_grid));
  *out = static_cast<const uint2*>(p);
  return 0;
}

// IQ2_S magnitude table (1024 rows), likewise.
__device__ uint2 g_iq2s_grid[1024];
static bool g_grid_s_ready[64] = {false};

int iq2s_grid(const uint2** out) {
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !g_grid_s_ready[dev])
    return fail(B2G_E_STATE, "IQ2_S grid not uploaded on device %d: call b2g_set_iq2s_grid first", dev);
  void* p = nullptr;
  B2G_CUDA_OK(cudaGetSymbolAddress(&p, g_iq2s_grid));
  *out = static_cast<const uint2*>(p);
  return 0;
}

}  // namespace b2g

extern "C" {

const char* b2g_last_error(void) { return b2g::last_error_buffer(); }
int b2g_abi_version(void) { return 1; }

int b2g_set_iq2xxs_grid(const uint8_t* host_grid_256x8) {
  B2G_REQUIRE(host_grid_256x8 != nullptr, "grid pointer is null");
  for (int i = 0; i < 2048; ++i) {
    const uint8_t v = host_grid_256x8[i];
    B2G_REQUIRE(v == 8 || v == 25 || v == 43, "grid byte %d has value %d, expected one of 8/25/43", i, (int)v);
  }
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  B2G_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  B2G_CUDA_OK(cudaMemcpyToSymbol(b2g::g_iq2xxs_grid, host_grid_256x8, 2048));
  b2g::g_grid_ready[dev] = true;
  return 0;
}

int b2g_set_iq2s_grid(const uint8_t* host_grid_1024x8) {
  B2G_REQUIRE(host_grid_1024x8 != nullptr, "grid pointer is null");
  for (int i = 0; i < 8192; ++i) {
    const uint8_t v = host_grid_1024x8[i];
    B2G_REQUIRE(v == 8 || v == 25 || v == 43, "grid byte %d has value %d, expected one of 8/25/43", i, (int)v);
  }
  int dev = 0;
  B2G_CUDA_OK(cudaGetDevice(&dev));
  B2G_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  B2G_CUDA_OK(cudaMemcpyToSymbol(b2g::g_iq2s_grid, host_grid_1024x8, 8192));
  b2g::g_grid_s_ready[dev] = true;
  return 0;
}

}  // extern "C"

// SMs that the persistent quantized GEMM leaves free (an even number: it runs on CTA pairs), for kernels of another stream
// that must not share an SM with it.  Process-wide, read at every GEMM launch.
namespace b2g {
static std::atomic<int> g_gemm_sm_margin{0};
int gemm_sm_margin() { return g_gemm_sm_margin.load(std::memory_order_relaxed); }
}  // namespace b2g

extern "C" int b2g_set_gemm_sm_margin(int sms) {
  B2G_REQUIRE(sms >= 0 && sms <= 64 && sms % 2 == 0, "gemm sm margin %d must be an even number between 0 and 64", sms);
  b2g::g_gemm_sm_margin.store(sms, std::memory_order_relaxed);
  return 0;
}
