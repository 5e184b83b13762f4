// Device-side decoders for the GGUF block formats on the path: Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ2_XXS, IQ2_S.
//
// The arithmetic reproduces the float32 decode of the public format definition bit for bit
// after the final bf16 round-to-nearest-even:
//   Q8_0    q * d                                 (19 significant bits: exact in fp32)
//   Q4_K    (d*sc)*q - (dmin*m)                   (both products exact; the subtraction rounds once,
//                                                  so a single fused multiply-add gives the same bits)
//   Q2_K    (d*s)*q - (dmin*m), s and m 4-bit    (as Q4_K: both products exact, one fused multiply-add)
//   Q3_K    (d*scale)*q, 6-bit scales, q in -4..3 (11 x 6, then x 3 significant bits: both products exact)
//   Q5_K    as Q4_K with a fifth bit per value    (products of 17 and 22 significant bits: exact)
//   Q6_K    (d*scale)*q                           (11 x 7, then x 6 significant bits: both products exact)
//   IQ2_XXS d*(0.5+s4)*0.25 * grid * sign         (22 significant bits: exact in fp32)
//   IQ2_S   the same with a 1024-row grid, explicit sign bytes and a sub-scale per 16 values
// Block layouts (bytes): Q8_0 34 = fp16 d | 32 x int8; Q4_K 144 = fp16 d | fp16 dmin | 12 scale bytes
// | 128 nibble bytes; Q2_K 84 = 16 scale bytes (scale | min << 4, one per 16 values) | 64 bytes of 2-bit values
// | fp16 d | fp16 dmin; Q3_K 110 = 32 mask bytes (bit g of byte l: group g, value l; CLEAR means minus 4) | 64 bytes of
// 2-bit values | 12 bytes of packed 6-bit scales | fp16 d; Q5_K 176 = the Q4_K header | 32 bytes of fifth bits (bit j of byte l: value l of sub-block j)
// | 128 nibble bytes; Q6_K 210 = 128 low-nibble bytes | 64 high-pair bytes | 16 int8 scales | fp16 d;
// IQ2_XXS 66 = fp16 d | 8 x (4 grid indices | u32: 4 x 7-bit signs + 4-bit scale); IQ2_S 82 = fp16 d | 32 index bytes
// | 32 sign bytes | 8 bytes of index bits 8-9 (four groups each) | 8 scale bytes (two nibbles, 16 values each).
#pragma once

#include "b2g_common.cuh"

namespace b2g {
namespace fmt {

template <int QT> struct Block;
template <> struct Block<B2G_Q8_0> { static constexpr int kValues = 32, kBytes = 34; };
template <> struct Block<B2G_Q4_K> { static constexpr int kValues = 256, kBytes = 144; };
template <> struct Block<B2G_IQ2_XXS> { static constexpr int kValues = 256, kBytes = 66; };
template <> struct Block<B2G_Q6_K> { static constexpr int kValues = 256, kBytes = 210; };
template <> struct Block<B2G_Q5_K> { static constexpr int kValues = 256, kBytes = 176; };
template <> struct Block<B2G_Q2_K> { static constexpr int kValues = 256, kBytes = 84; };
template <> struct Block<B2G_Q3_K> { static constexpr int kValues = 256, kBytes = 110; };
template <> struct Block<B2G_IQ2_S> { static constexpr int kValues = 256, kBytes = 82; };

__host__ __device__ inline int64_t row_bytes(int qtype, int64_t k) {
  switch (qtype) {
    case B2G_Q8_0: return k / 32 * 34;
    case B2G_Q4_K: return k / 256 * 144;
    case B2G_IQ2_XXS: return k / 256 * 66;
    case B2G_Q6_K: return k / 256 * 210;
    case B2G_Q5_K: return k / 256 * 176;
    case B2G_Q2_K: return k / 256 * 84;
    case B2G_Q3_K: return k / 256 * 110;
    case B2G_IQ2_S: return k / 256 * 82;
    default: return -1;
  }
}
__host__ __device__ inline int block_values(int qtype) { return qtype == B2G_Q8_0 ? 32 : 256; }

// Exact small-integer -> float: place the byte in the mantissa of 2^23 and subtract 2^23.
__device__ __forceinline__ float byte_to_float(uint32_t word, int byte_index) {
  // selector nibbles (lsb first): result byte0 = word.byte[i], byte1 = 0x00, byte2 = 0x00, byte3 = 0x4B
  const uint32_t magic = __byte_perm(word, 0x4B000000u, 0x7540u + byte_index);
  return __uint_as_float(magic) - 8388608.0f;
}

// Q4_K: 6-bit (scale, min) of sub-block `i` (0..7) from the 12 scale bytes held as three words.
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int i, uint32_t& sc, uint32_t& mn) {
  const int sh = (i & 3) * 8;
  const uint32_t a = (s0 >> sh) & 0xFFu, m = (s1 >> sh) & 0xFFu, lo = (s2 >> sh) & 0xFFu;
  if (i < 4) {
    sc = a & 63u;
    mn = m & 63u;
  } else {
    sc = (lo & 15u) | ((a >> 6) << 4);
    mn = (lo >> 4) | ((m >> 6) << 4);
  }
}

// IQ2_XXS: sign byte of a 7-bit index (bit 7 = parity of the low seven bits).
__device__ __forceinline__ uint32_t iq2_sign_byte(uint32_t idx7) { return idx7 | ((__popc(idx7) & 1u) << 7); }

// ---- decode 8 consecutive values k0..k0+7 (k0 % 8 == 0) of one packed row in GLOBAL memory ----
// Used by the stand-alone dequantiser; the GEMM kernels decode from shared memory instead.
template <int QT>
struct Decode8;

template <>
struct Decode8<B2G_Q8_0> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 5) * 34;  // 34-byte blocks are only 2-byte aligned
    const float d = dev::half_bits_to_float(*reinterpret_cast<const unsigned short*>(b));
    const unsigned short* q = reinterpret_cast<const unsigned short*>(b + 2 + (k0 & 31));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t two = q[i];
      const float lo = static_cast<float>(static_cast<int>(static_cast<signed char>(two & 0xFF)));
      const float hi = static_cast<float>(static_cast<int>(static_cast<signed char>(two >> 8)));
      v[2 * i] = __fmul_rn(lo, d);
      v[2 * i + 1] = __fmul_rn(hi, d);
    }
  }
};

template <>
struct Decode8<B2G_Q4_K> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 144;  // 144-byte blocks keep 16-byte alignment
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);
    const int within = k0 & 255;
    const int sub = within >> 5;               // sub-block 0..7
    uint32_t sc, mn;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, sub, sc, mn);
    const float dsc = __fmul_rn(dev::half_bits_to_float(hdr.x), static_cast<float>(sc));
    const float dm = __fmul_rn(dev::half_bits_to_float(hdr.x >> 16), static_cast<float>(mn));
    // sub-blocks 2j / 2j+1 share 32 bytes: low / high nibbles
    const uint2 w = *reinterpret_cast<const uint2*>(b + 16 + (sub >> 1) * 32 + (within & 31));
    const int shift = (sub & 1) * 4;
    const uint32_t w0 = (w.x >> shift) & 0x0F0F0F0Fu, w1 = (w.y >> shift) & 0x0F0F0F0Fu;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fmaf_rn(dsc, byte_to_float(w0, i), -dm);
      v[4 + i] = __fmaf_rn(dsc, byte_to_float(w1, i), -dm);
    }
  }
};

template <>
struct Decode8<B2G_Q2_K> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 84;   // 84-byte blocks are 4-byte aligned
    const int within = k0 & 255;
    const int h = within >> 7, t = (within >> 5) & 3, l = within & 31;   // half, 32-value group, position (multiple of 8)
    const uint32_t s = b[within >> 4];
    const uint32_t dd = *reinterpret_cast<const uint32_t*>(b + 80);
    const float dl = __fmul_rn(dev::half_bits_to_float(dd), static_cast<float>(s & 15u));
    const float ml = __fmul_rn(dev::half_bits_to_float(dd >> 16), static_cast<float>(s >> 4));
    const uint32_t* qs = reinterpret_cast<const uint32_t*>(b + 16 + 32 * h + l);
#pragma unroll
    for (int w2 = 0; w2 < 2; ++w2) {
      const uint32_t q = (qs[w2] >> (2 * t)) & 0x03030303u;
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * w2 + i] = __fmaf_rn(dl, byte_to_float(q, i), -ml);
    }
  }
};

// Three-bit value (0..7) minus 4 / six-bit value minus 32 at byte i of `word` -> exact float.
__device__ __forceinline__ float q3_to_float(uint32_t word, int i) {
  const uint32_t magic = __byte_perm(word, 0x4B000000u, 0x7540u + i);
  return __uint_as_float(magic) - 8388612.0f;  // 2^23 + 4
}
__device__ __forceinline__ float q6_to_float(uint32_t word, int i) {
  const uint32_t magic = __byte_perm(word, 0x4B000000u, 0x7540u + i);
  return __uint_as_float(magic) - 8388640.0f;  // 2^23 + 32
}

template <>
struct Decode8<B2G_Q3_K> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 110;  // 110-byte blocks are only 2-byte aligned
    const int within = k0 & 255;
    const int h = within >> 7, t = (within >> 5) & 3, l = within & 31, g = 4 * h + t, i = within >> 4;
    const unsigned short* qs = reinterpret_cast<const unsigned short*>(b + 32 + 32 * h + l);
    const unsigned short* hm = reinterpret_cast<const unsigned short*>(b + l);
    const uint32_t s6 = ((static_cast<uint32_t>(b[96 + (i & 7)]) >> (4 * (i >> 3))) & 15u) |
                        (((static_cast<uint32_t>(b[104 + (i & 3)]) >> (2 * (i >> 2))) & 3u) << 4);
    const float d = dev::half_bits_to_float(*reinterpret_cast<const unsigned short*>(b + 108));
    const float dl = __fmul_rn(d, static_cast<float>(static_cast<int>(s6) - 32));
#pragma unroll
    for (int w2 = 0; w2 < 2; ++w2) {
      const uint32_t qw = static_cast<uint32_t>(qs[2 * w2]) | (static_cast<uint32_t>(qs[2 * w2 + 1]) << 16);
      const uint32_t hw = static_cast<uint32_t>(hm[2 * w2]) | (static_cast<uint32_t>(hm[2 * w2 + 1]) << 16);
      const uint32_t q = ((qw >> (2 * t)) & 0x03030303u) | (((hw >> g) & 0x01010101u) << 2);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[4 * w2 + e] = __fmul_rn(dl, q3_to_float(q, e));
    }
  }
};

template <>
struct Decode8<B2G_Q5_K> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 176;  // 176-byte blocks keep 16-byte alignment
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);
    const int within = k0 & 255;
    const int sub = within >> 5;               // sub-block 0..7
    uint32_t sc, mn;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, sub, sc, mn);
    const float dsc = __fmul_rn(dev::half_bits_to_float(hdr.x), static_cast<float>(sc));
    const float dm = __fmul_rn(dev::half_bits_to_float(hdr.x >> 16), static_cast<float>(mn));
    const uint2 hb = *reinterpret_cast<const uint2*>(b + 16 + (within & 31));
    const uint2 w = *reinterpret_cast<const uint2*>(b + 48 + (sub >> 1) * 32 + (within & 31));
    const int shift = (sub & 1) * 4;
    const uint32_t w0 = ((w.x >> shift) & 0x0F0F0F0Fu) | (((hb.x >> sub) & 0x01010101u) << 4);
    const uint32_t w1 = ((w.y >> shift) & 0x0F0F0F0Fu) | (((hb.y >> sub) & 0x01010101u) << 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fmaf_rn(dsc, byte_to_float(w0, i), -dm);
      v[4 + i] = __fmaf_rn(dsc, byte_to_float(w1, i), -dm);
    }
  }
};

template <>
struct Decode8<B2G_Q6_K> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2*, float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 210;  // 210-byte blocks are only 2-byte aligned
    const int within = k0 & 255;
    const int h = within >> 7, t = (within >> 5) & 3, l = within & 31;   // half, 32-value group, position (multiple of 8)
    const unsigned short* ql = reinterpret_cast<const unsigned short*>(b + 64 * h + 32 * (t & 1) + l);
    const unsigned short* qh = reinterpret_cast<const unsigned short*>(b + 128 + 32 * h + l);
    const float d = dev::half_bits_to_float(*reinterpret_cast<const unsigned short*>(b + 208));
    const float sc = static_cast<float>(static_cast<int>(static_cast<signed char>(b[192 + (within >> 4)])));
    const float dsc = __fmul_rn(d, sc);
    const int lo_shift = (t >> 1) * 4, hi_shift = 2 * t;
#pragma unroll
    for (int w2 = 0; w2 < 2; ++w2) {
      const uint32_t lw = static_cast<uint32_t>(ql[2 * w2]) | (static_cast<uint32_t>(ql[2 * w2 + 1]) << 16);
      const uint32_t hw = static_cast<uint32_t>(qh[2 * w2]) | (static_cast<uint32_t>(qh[2 * w2 + 1]) << 16);
      const uint32_t q = ((lw >> lo_shift) & 0x0F0F0F0Fu) | (((hw >> hi_shift) & 0x03030303u) << 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * w2 + i] = __fmul_rn(dsc, q6_to_float(q, i));
    }
  }
};

template <>
struct Decode8<B2G_IQ2_XXS> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2* __restrict__ grid,
                                             float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 66;   // 66-byte blocks are only 2-byte aligned
    const unsigned short* h = reinterpret_cast<const unsigned short*>(b);
    const float d = dev::half_bits_to_float(h[0]);
    const int within = k0 & 255;
    const int grp = within >> 5;               // group of 32 values: 8 bytes at 2 + 8*grp
    const int sub = (within >> 3) & 3;         // which 8-value row of the group
    const unsigned short* g = h + 1 + grp * 4;
    const uint32_t idx4 = static_cast<uint32_t>(g[0]) | (static_cast<uint32_t>(g[1]) << 16);
    const uint32_t word = static_cast<uint32_t>(g[2]) | (static_cast<uint32_t>(g[3]) << 16);
    const float db = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(word >> 28)), 0.25f);
    const uint32_t signs = iq2_sign_byte((word >> (7 * sub)) & 127u);
    const uint2 mag = grid[(idx4 >> (8 * sub)) & 255u];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t m = ((i < 4 ? mag.x : mag.y) >> (8 * (i & 3))) & 0xFFu;
      const float mv = __fmul_rn(db, static_cast<float>(m));
      v[i] = ((signs >> i) & 1u) ? -mv : mv;
    }
  }
};

template <>
struct Decode8<B2G_IQ2_S> {
  __device__ static __forceinline__ void run(const uint8_t* __restrict__ row, int k0, const uint2* __restrict__ grid,
                                             float (&v)[8]) {
    const uint8_t* b = row + (k0 >> 8) * 82;   // 82-byte blocks are only 2-byte aligned
    const int c = (k0 & 255) >> 3;             // group of 8 values, 0..31
    const float d = dev::half_bits_to_float(*reinterpret_cast<const unsigned short*>(b));
    const uint32_t idx = static_cast<uint32_t>(b[2 + c]) | (((static_cast<uint32_t>(b[66 + (c >> 2)]) >> (2 * (c & 3))) & 3u) << 8);
    const uint32_t signs = b[34 + c];
    const uint32_t s4 = (static_cast<uint32_t>(b[74 + (c >> 2)]) >> (4 * ((c >> 1) & 1))) & 15u;
    const float db = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(s4)), 0.25f);
    const uint2 mag = grid[idx];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t m = ((i < 4 ? mag.x : mag.y) >> (8 * (i & 3))) & 0xFFu;
      const float mv = __fmul_rn(db, static_cast<float>(m));
      v[i] = ((signs >> i) & 1u) ? -mv : mv;
    }
  }
};

}  // namespace fmt
}  // namespace b2g
