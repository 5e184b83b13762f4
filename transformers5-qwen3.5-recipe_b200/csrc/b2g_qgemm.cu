// Quantized-weight GEMM for sm_100a: activations by TMA, packed GGUF blocks by TMA in their on-disk
// layout, unpack to bf16 in shared memory, tcgen05.mma with fp32 accumulators in TMEM.
//
// One persistent, warp-specialised kernel serves four entry points:
//   dense   forward   Y[M,N]  = X[M,K] . deq(W[N,K])^T                 (+ bias, + LoRA)
//   dense   dgrad     dX[M,K] = dY[M,N] . deq(W[N,K])                  (+ LoRA)
//   grouped forward   per ragged expert segment, one or two (gate, up) weight tensors
//   grouped dgrad     per segment, one or two gradient/weight pairs summed in one accumulator
//
// CTAs work in PAIRS (a cluster of two, tcgen05 cta_group::2).  A pair owns a tile of up to 512 rows x
// 256 output columns: each MMA is 256 x 256 x 16 across the pair, each CTA holding 128 of its rows in
// TMEM, and two such row blocks (MT = 2) share every unpacked weight tile.  Per reduction step of 64 a
// CTA holds
//   A  : MT x [128 rows x 64] bf16, 128-byte swizzle, written by TMA          (A operand, K-major)
//   B  : ITS HALF of the weight tile, 128-byte swizzled bf16 written by its unpack warps:
//        forward: [128 W rows x 64 k]       -> B operand K-major  (N = W rows, K = k)
//        dgrad  : 2 x [64 W rows x 64 k]    -> B operand MN-major (N = k,      K = W rows)
//        The unpack warps write the same [w_row][k] layout in both directions; only the shared-memory
//        descriptors differ, so no packed transpose is ever built.
// so each packed block is unpacked once per 512 rows, and each CTA reads only half of B from its own
// shared memory.  The LoRA up-projection is one extra K=16 MMA per row block on 32-byte-swizzled tiles.
//
// Warp roles (736 threads per CTA): 0 = activation / LoRA tile producer (TMA), 1 = MMA issuer (first CTA of the
// pair only) + TMEM owner, 2-5 = epilogue (TMEM -> registers -> 32-byte global stores), 6-21 = unpack in four groups that take
// reduction steps round-robin (four steps in flight), 22 = packed-weight producer (TMA).  Barriers that gate the MMA
// (A / B / LoRA tiles ready, accumulator drained) live in the first CTA and collect arrivals from both;
// barriers that release buffers are signalled in both CTAs by tcgen05.commit.  No TMA multicast is used:
// every CTA loads its own tiles.  All mbarrier waits are bounded.
#include "b2g_formats.cuh"

namespace b2g {
int gemm_sm_margin();
int iq2xxs_grid(const uint2** out);
int iq2s_grid(const uint2** out);

namespace qg {

constexpr int kFwd = 0, kDgrad = 1;
constexpr int kBM = 128;          // rows per CTA and row block
constexpr int kPairRows = 256;    // rows per row block across the pair
constexpr int kBN = 256;          // output columns per tile (MMA N across the pair)
constexpr int kBNh = 128;         // of which this CTA unpacks / holds
constexpr int kBK = 64;           // reduction step
constexpr int kMT = 2;            // row blocks per tile
constexpr int kTileRows = kPairRows * kMT;  // 512
constexpr int kATile = kBM * kBK * 2;       // 16384
constexpr int kBStage = kBNh * kBK * 2;     // 16384
constexpr int kBStages = 4;
constexpr int kUnpackWarps = 16;
constexpr int kUnpackGroups = 4;            // groups take reduction steps round-robin, so four steps are unpacked concurrently
constexpr int kGroupWarps = kUnpackWarps / kUnpackGroups;
constexpr int kGroupThreads = 32 * kGroupWarps;   // 128 threads: one 64-value slice of a W row each
static_assert(kGroupThreads == 128, "the unpack mapping assumes 128 threads per group");
constexpr int kThreads = 32 * (7 + kUnpackWarps);  // + A producer, MMA, 4 epilogue, packed-weight producer
constexpr int kLoraATile = kBM * 32;        // [128 x 16] bf16
constexpr int kLoraBTile = kBNh * 32;       // 4096 either way
constexpr int kTmemCols = 512;

// Packed-stage geometry: what one reduction step needs of the packed weight in ONE CTA, as TMA boxes over
// the payload viewed as uint32 [rows, pitch/4].  x coordinates are always multiples of 4 words (16 bytes).
template <int QT, int MODE> struct Packed;
// Q4_K forward: header (d, dmin, 12 scale bytes) + the 32 nibble bytes of one 64-value pair, as
// three [128 rows x 16 B] boxes so that each thread reads its row with conflict-free 16-byte loads.
template <> struct Packed<B2G_Q4_K, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 3 * 2048, kSteps = 1; };
// Q4_K dgrad: whole 144-byte super-blocks of 64 rows (row stride 144 B: conflict-free 16-byte loads);
// each CTA decodes the two 64-value pairs of its 128 columns.
template <> struct Packed<B2G_Q4_K, kDgrad> { static constexpr int kBoxWords = 36, kBoxRows = 64, kBytes = 64 * 144, kSteps = 1; };
// Q8_0 forward: two 34-byte blocks start at byte 68*step; an 80-byte window from the 16-byte boundary below
// covers them (the start is at most 12 bytes into the window).
template <> struct Packed<B2G_Q8_0, kFwd> { static constexpr int kBoxWords = 20, kBoxRows = 128, kBytes = 128 * 80, kSteps = 1; };
// Q8_0 dgrad: this CTA's 128 columns are four blocks (136 B) starting at byte 272*tile + 136*rank of the row; a
// 144-byte window from the 16-byte boundary below covers them (the start is 0 or 8 bytes into the window).
template <> struct Packed<B2G_Q8_0, kDgrad> { static constexpr int kBoxWords = 36, kBoxRows = 64, kBytes = 64 * 144, kSteps = 1; };
// IQ2_XXS: 66-byte super-blocks are not 16-byte aligned; an 80-byte window from the boundary below covers one
// (the start is at most 14 bytes into the window).
template <> struct Packed<B2G_IQ2_XXS, kFwd> { static constexpr int kBoxWords = 20, kBoxRows = 128, kBytes = 128 * 80, kSteps = 1; };
template <> struct Packed<B2G_IQ2_XXS, kDgrad> { static constexpr int kBoxWords = 20, kBoxRows = 64, kBytes = 64 * 80, kSteps = 1; };
// Q2_K: 84-byte super-blocks start on a multiple of 4 bytes of a 16-byte line.  A 64-value step uses 32 bytes of 2-bit values
// (shared with the other step of the same 128-value half), four scale bytes and d | dmin: six 16-byte pieces per row with
// the slack of the alignment (two from the line below the scales, three below the values, one holding d | dmin).  As for
// Q6_K one forward slot serves the two steps that read the same bytes.
template <> struct Packed<B2G_Q2_K, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 6 * 2048, kSteps = 2; };
template <> struct Packed<B2G_Q2_K, kDgrad> { static constexpr int kBoxWords = 4, kBoxRows = 64, kBytes = 6 * 1024, kSteps = 1; };
// Q3_K: 110-byte super-blocks start on any even byte.  A step uses the 32 mask bytes, 32 bytes of 2-bit values (shared with
// the other step of its half), the 12 scale bytes and d: eight pieces per row with the slack (three below the mask, three
// below the values, two below the scales).  Forward slots serve step pairs as for Q6_K.
template <> struct Packed<B2G_Q3_K, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 8 * 2048, kSteps = 2; };
template <> struct Packed<B2G_Q3_K, kDgrad> { static constexpr int kBoxWords = 4, kBoxRows = 64, kBytes = 8 * 1024, kSteps = 1; };
// IQ2_S: 82-byte super-blocks on even bytes; a 96-byte window from the 16-byte boundary below covers one, as six pieces per
// row.  A step needs 8 index bytes, 8 sign bytes and a few bits more of its super-block; the whole window is loaded (it is
// small) and, forward, shared by the two steps of a pair (the other pair of the super-block loads it again).
template <> struct Packed<B2G_IQ2_S, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 6 * 2048, kSteps = 2; };
template <> struct Packed<B2G_IQ2_S, kDgrad> { static constexpr int kBoxWords = 4, kBoxRows = 64, kBytes = 6 * 1024, kSteps = 1; };
// Q5_K: 176-byte super-blocks keep 16-byte alignment like Q4_K.  Forward: header, the 32 bytes of fifth bits (all eight
// sub-blocks share them) and the 32 nibble bytes of one 64-value pair, as five [128 rows x 16 B] boxes.  Dgrad: whole
// super-blocks of 64 rows (row stride 176 B = 11 x 16: conflict-free 16-byte loads).
template <> struct Packed<B2G_Q5_K, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 5 * 2048, kSteps = 1; };
template <> struct Packed<B2G_Q5_K, kDgrad> { static constexpr int kBoxWords = 44, kBoxRows = 64, kBytes = 64 * 176, kSteps = 1; };
// Q6_K: 210-byte super-blocks start on any even byte of a 16-byte line.  A 64-value step uses, of its super-block, 64 bytes
// of low nibbles, 32 bytes of high bit pairs, 4 scales and d; with the slack of the alignment that is ten 16-byte pieces
// per row: five from the line below the nibbles, three below the bit pairs, two below the scales.  Each piece is one
// [rows x 16 B] box, so threads read their row's pieces without bank conflicts.  Forward: steps 2m and 2m+1 use the SAME
// bytes (low / high nibbles, bit pairs 0-3 / 4-7), so one slot serves both and the two unpack groups that take them.
template <> struct Packed<B2G_Q6_K, kFwd> { static constexpr int kBoxWords = 4, kBoxRows = 128, kBytes = 10 * 2048, kSteps = 2; };
template <> struct Packed<B2G_Q6_K, kDgrad> { static constexpr int kBoxWords = 4, kBoxRows = 64, kBytes = 10 * 1024, kSteps = 1; };

template <int QT, int MODE>
struct Cfg {
  using P = Packed<QT, MODE>;
  static constexpr int kAStages = 3;
  static constexpr int kAStage = kMT * kATile;
  // packed slots: slot s always belongs to the same unpack group(s) (P::kSteps consecutive groups share one), so each group
  // sees every phase of its barriers
  static constexpr int kPStages = kUnpackGroups / P::kSteps;
  static_assert(kBStages == kUnpackGroups, "B slots are owned by unpack groups as well");
  static constexpr int kPStage = (P::kBytes + 1023) / 1024 * 1024;
  // shared-memory map (offsets from a 1024-byte aligned base)
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kAStages * kAStage;
  static constexpr int kOffP = kOffB + kBStages * kBStage;
  static constexpr int kOffLA = kOffP + kPStages * kPStage;
  static constexpr int kOffLB = kOffLA + kMT * kLoraATile;
  static constexpr int kGridRows = QT == B2G_IQ2_XXS ? 256 : (QT == B2G_IQ2_S ? 1024 : 0);   // magnitude table of the IQ2 types
  static constexpr int kOffGrid = kOffLB + kLoraBTile;
  static constexpr int kOffBar = kOffGrid + 8 * kGridRows;
  // "released" barriers: one per reduction step, in a ring whose length both buffer rings divide, so that the A producer (its
  // stage was last used kAStages steps ago) and the unpack groups (kBStages steps ago) wait on the same arrival
  static constexpr int kRelBars = 12;
  static_assert(kRelBars % kAStages == 0 && kRelBars % kBStages == 0, "release ring must be a multiple of both buffer rings");
  static constexpr int kNumBars = kAStages + kBStages + kRelBars + 2 * kPStages + 2 + 3;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;                   // tmem slot, abort flag
  // forward only, where the budget allows: one [32 rows x 64 columns] bf16 staging tile (128B swizzle) per epilogue warp,
  // from which finished accumulator chunks leave as bulk tensor stores
  static constexpr int kOffStage = (kOffMisc + 16 + 1023) / 1024 * 1024;
  static constexpr int kStageWarp = 32 * 128;
  static constexpr bool kStaged = MODE == kFwd && kOffStage + 4 * kStageWarp + 1024 <= 232448;
  static constexpr int kSmemBytes = kStaged ? kOffStage + 4 * kStageWarp + 1024 : kOffMisc + 16 + 1024;   // + alignment slack
  static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

struct Params {
  int m_total;        // activation rows (M, or all routed rows R)
  int n;              // W rows per expert and per payload
  int k;              // W logical columns
  int nseg;           // payload tensors (1, or 2 for gate|up)
  int num_ct;         // output column tiles
  int ct_per_seg;     // forward: column tiles per payload
  int num_iters;      // reduction steps per tile
  int iters_per_seg;  // dgrad: steps per payload
  int dense_m_tiles;  // dense only
  int has_lora;
  int lora_rows;      // forward: rows per expert of the padded LoRA-B tensor
  int ldc;
  const int4* tiles;  // grouped: [0] = {count, rows_per_tile, ..}, [1..] = {expert, row0, rows, _}
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  const __nv_bfloat16* bias;
  const uint2* grid;  // IQ2_XXS table in global memory
  int* status;
  int wide_ok;        // output rows and row segments start on 32-byte boundaries
  int tma_out;        // the output tensor maps are valid (forward, 16-byte aligned rows)
  uint32_t spin_limit;   // polls the unpack warps' wait for packed bytes (site 401) may take before the kernel gives up; every
                         // other wait keeps the library's limit and leaves as soon as it sees the CTA's abort flag
  int hold_weights;      // test hook: the packed-weight producer issues nothing, so the unpack warps' wait (site 401) must run out
};

struct Tile { int expert, row0, rows, ct; };

__device__ __forceinline__ int num_m_tiles(const Params& p) { return p.tiles ? p.tiles[0].x : p.dense_m_tiles; }

__device__ __forceinline__ Tile get_tile(const Params& p, int item) {
  Tile t;
  const int mt = item / p.num_ct;
  t.ct = item - mt * p.num_ct;
  if (p.tiles) {
    const int4 e = p.tiles[1 + mt];
    t.expert = e.x; t.row0 = e.y; t.rows = e.z;
  } else {
    t.expert = 0; t.row0 = mt * kTileRows;
    const int left = p.m_total - t.row0;
    t.rows = left < kTileRows ? left : kTileRows;
  }
  return t;
}

// ------------------------------------------------------------------------------------------------
// Row decoders.  One unpack thread owns 32 consecutive values of one W row per reduction step (half of
// the 64-value slice): out[4*c + i] holds values 8c+2i, 8c+2i+1 of its half as a bf16 pair, chunk c being
// one 16-byte shared-memory vector.  `half` is uniform across a warp.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void q4k_half(const uint4 hdr, const uint4 qa, const uint4 qb, int pair, int half, uint32_t (&out)[16]) {
  uint32_t sc, mn;
  fmt::q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pair + half, sc, mn);
  const float dsc = __fmul_rn(dev::half_bits_to_float(hdr.x), static_cast<float>(sc));
  const float ndm = -__fmul_rn(dev::half_bits_to_float(hdr.x >> 16), static_cast<float>(mn));
  const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
  const int shift = 4 * half;  // sub-block 2*pair lives in the low nibbles, 2*pair+1 in the high nibbles
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q = (w[i] >> shift) & 0x0F0F0F0Fu;  // bytes 4i..4i+3 -> values 4i..4i+3 of the sub-block
    out[2 * i] = dev::pack_bf16(__fmaf_rn(dsc, fmt::byte_to_float(q, 0), ndm), __fmaf_rn(dsc, fmt::byte_to_float(q, 1), ndm));
    out[2 * i + 1] = dev::pack_bf16(__fmaf_rn(dsc, fmt::byte_to_float(q, 2), ndm), __fmaf_rn(dsc, fmt::byte_to_float(q, 3), ndm));
  }
}

// Q5_K: as q4k_half with the fifth bit of value l of sub-block j taken from bit j of the l-th fifth-bit byte.
__device__ __forceinline__ void q5k_half(const uint4 hdr, const uint4 qa, const uint4 qb, const uint4 ha, const uint4 hb, int pair, int half,
                                         uint32_t (&out)[16]) {
  uint32_t sc, mn;
  const int sub = 2 * pair + half;
  fmt::q4k_scale_min(hdr.y, hdr.z, hdr.w, sub, sc, mn);
  const float dsc = __fmul_rn(dev::half_bits_to_float(hdr.x), static_cast<float>(sc));
  const float ndm = -__fmul_rn(dev::half_bits_to_float(hdr.x >> 16), static_cast<float>(mn));
  const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
  const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
  const int shift = 4 * half;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q = ((w[i] >> shift) & 0x0F0F0F0Fu) | (((h[i] >> sub) & 0x01010101u) << 4);
    out[2 * i] = dev::pack_bf16(__fmaf_rn(dsc, fmt::byte_to_float(q, 0), ndm), __fmaf_rn(dsc, fmt::byte_to_float(q, 1), ndm));
    out[2 * i + 1] = dev::pack_bf16(__fmaf_rn(dsc, fmt::byte_to_float(q, 2), ndm), __fmaf_rn(dsc, fmt::byte_to_float(q, 3), ndm));
  }
}

// int8 (already XOR 0x80 per byte) at byte i of `word` -> exact float
__device__ __forceinline__ float sbyte_to_float(uint32_t word_x80, int i) {
  const uint32_t magic = __byte_perm(word_x80, 0x4B000000u, 0x7540u + i);
  return __uint_as_float(magic) - 8388736.0f;  // 2^23 + 128
}

// One of two consecutive Q8_0 blocks (68 bytes, given as 17 words from the first block's scale).
__device__ __forceinline__ void q8_half(const uint32_t (&w)[17], int half, uint32_t (&out)[16]) {
  if (half == 0) {
    const float d = dev::half_bits_to_float(w[0]);  // bytes 0-1; values at bytes 2..33 straddle words
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t a = __byte_perm(w[2 * c], w[2 * c + 1], 0x5432) ^ 0x80808080u;
      const uint32_t b = __byte_perm(w[2 * c + 1], w[2 * c + 2], 0x5432) ^ 0x80808080u;
      out[4 * c + 0] = dev::pack_bf16(__fmul_rn(sbyte_to_float(a, 0), d), __fmul_rn(sbyte_to_float(a, 1), d));
      out[4 * c + 1] = dev::pack_bf16(__fmul_rn(sbyte_to_float(a, 2), d), __fmul_rn(sbyte_to_float(a, 3), d));
      out[4 * c + 2] = dev::pack_bf16(__fmul_rn(sbyte_to_float(b, 0), d), __fmul_rn(sbyte_to_float(b, 1), d));
      out[4 * c + 3] = dev::pack_bf16(__fmul_rn(sbyte_to_float(b, 2), d), __fmul_rn(sbyte_to_float(b, 3), d));
    }
  } else {
    const float d = dev::half_bits_to_float(w[8] >> 16);  // bytes 34-35; values at bytes 36..67, word aligned
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t e = w[9 + 2 * c] ^ 0x80808080u, f = w[10 + 2 * c] ^ 0x80808080u;
      out[4 * c + 0] = dev::pack_bf16(__fmul_rn(sbyte_to_float(e, 0), d), __fmul_rn(sbyte_to_float(e, 1), d));
      out[4 * c + 1] = dev::pack_bf16(__fmul_rn(sbyte_to_float(e, 2), d), __fmul_rn(sbyte_to_float(e, 3), d));
      out[4 * c + 2] = dev::pack_bf16(__fmul_rn(sbyte_to_float(f, 0), d), __fmul_rn(sbyte_to_float(f, 1), d));
      out[4 * c + 3] = dev::pack_bf16(__fmul_rn(sbyte_to_float(f, 2), d), __fmul_rn(sbyte_to_float(f, 3), d));
    }
  }
}

// Read `N` words starting at byte offset `off` (a multiple of 4, < 16) of a 16-byte aligned row.
template <int N>
__device__ __forceinline__ void load_words_shifted(uint32_t row16, int off, uint32_t (&w)[N]) {
  constexpr int kVec = (N + 3 + 3) / 4;  // enough 16-byte vectors for any shift
  uint32_t raw[kVec * 4];
#pragma unroll
  for (int v = 0; v < kVec; ++v) {
    const uint4 q = dev::lds128(row16 + 16 * v);
    raw[4 * v] = q.x; raw[4 * v + 1] = q.y; raw[4 * v + 2] = q.z; raw[4 * v + 3] = q.w;
  }
  const int s = off >> 2;  // warp-uniform
  if (s == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = raw[i];
  } else if (s == 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = raw[i + 1];
  } else if (s == 2) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = raw[i + 2];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = raw[i + 3];
  }
}

// IQ2_XXS: one 8-byte group (32 values): four grid-row indices and the sign/scale word.
__device__ __forceinline__ void iq2_half(float d, uint32_t idx4, uint32_t word, uint32_t grid_s, uint32_t (&out)[16]) {
  const float db = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(word >> 28)), 0.25f);
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint2 mag = dev::lds64(grid_s + (((idx4 >> (8 * s)) & 255u) << 3));
    const uint32_t sg = fmt::iq2_sign_byte((word >> (7 * s)) & 127u);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float m = __fmul_rn(db, fmt::byte_to_float(i < 4 ? mag.x : mag.y, i & 3));
      v[i] = __uint_as_float(__float_as_uint(m) ^ (((sg >> i) & 1u) << 31));
    }
    out[4 * s + 0] = dev::pack_bf16(v[0], v[1]);
    out[4 * s + 1] = dev::pack_bf16(v[2], v[3]);
    out[4 * s + 2] = dev::pack_bf16(v[4], v[5]);
    out[4 * s + 3] = dev::pack_bf16(v[6], v[7]);
  }
}

// `N` words that start `sft` bytes (even, < 16, warp-uniform) into the 16-byte aligned words `raw`.
template <int N, int NRAW>
__device__ __forceinline__ void extract_words(const uint32_t (&raw)[NRAW], int sft, uint32_t (&w)[N]) {
  static_assert(N + 3 <= NRAW, "not enough loaded words for the largest shift");
  const int ws = sft >> 2;
  const uint32_t bs = static_cast<uint32_t>(sft & 3) * 8u;   // 0 or 16 bits
  auto at = [&](int i) { return i < NRAW ? raw[i < NRAW ? i : 0] : 0u; };
  if (ws == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(at(i), at(i + 1), bs);
  } else if (ws == 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(at(i + 1), at(i + 2), bs);
  } else if (ws == 2) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(at(i + 2), at(i + 3), bs);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(at(i + 3), at(i + 4), bs);
  }
}

// Q2_K: 32 values of a 64-value slice; `j` = which quarter of the super-block (its parity picks bit pairs 0-1 or 2-3 of the
// bytes), `half` = first or second 32 values (the next bit pair).  value = fma(d * scale, q, -(dmin * min)).
__device__ __forceinline__ void q2k_half(const uint32_t (&qs)[8], uint32_t sc4, uint32_t dd, int j, int half, uint32_t (&out)[16]) {
  const float d = dev::half_bits_to_float(dd), dmin = dev::half_bits_to_float(dd >> 16);
  const uint32_t s0 = (sc4 >> (16 * half)) & 0xFFu, s1 = (sc4 >> (16 * half + 8)) & 0xFFu;   // scale bytes of values 0-15, 16-31
  const float dl0 = __fmul_rn(d, static_cast<float>(s0 & 15u)), nm0 = -__fmul_rn(dmin, static_cast<float>(s0 >> 4));
  const float dl1 = __fmul_rn(d, static_cast<float>(s1 & 15u)), nm1 = -__fmul_rn(dmin, static_cast<float>(s1 >> 4));
  const int shift = 4 * (j & 1) + 2 * half;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q = (qs[i] >> shift) & 0x03030303u;
    const float dl = i < 4 ? dl0 : dl1, nm = i < 4 ? nm0 : nm1;
    out[2 * i] = dev::pack_bf16(__fmaf_rn(dl, fmt::byte_to_float(q, 0), nm), __fmaf_rn(dl, fmt::byte_to_float(q, 1), nm));
    out[2 * i + 1] = dev::pack_bf16(__fmaf_rn(dl, fmt::byte_to_float(q, 2), nm), __fmaf_rn(dl, fmt::byte_to_float(q, 3), nm));
  }
}

// Q3_K: 32 values of a 64-value slice; `j` = which quarter of the super-block, `half` = first or second 32 values.  Group
// number g = 2j + half selects the mask bit, its parity within the half the bit pair of the value bytes.
__device__ __forceinline__ void q3k_half(const uint32_t (&hm)[8], const uint32_t (&qs)[8], uint32_t sc_lo, uint32_t sc_hi, float d, int j,
                                         int half, uint32_t (&out)[16]) {
  const uint32_t s6 = ((sc_lo >> (4 * (j >> 1))) & 0x0F0F0F0Fu) | (((sc_hi >> (2 * j)) & 0x03030303u) << 4);   // scales 4j .. 4j+3, plus 32
  const float dl0 = __fmul_rn(d, half ? fmt::q6_to_float(s6, 2) : fmt::q6_to_float(s6, 0));
  const float dl1 = __fmul_rn(d, half ? fmt::q6_to_float(s6, 3) : fmt::q6_to_float(s6, 1));
  const int g = 2 * j + half, shift = 2 * (g & 3);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q = ((qs[i] >> shift) & 0x03030303u) | (((hm[i] >> g) & 0x01010101u) << 2);
    const float dl = i < 4 ? dl0 : dl1;
    out[2 * i] = dev::pack_bf16(__fmul_rn(dl, fmt::q3_to_float(q, 0)), __fmul_rn(dl, fmt::q3_to_float(q, 1)));
    out[2 * i + 1] = dev::pack_bf16(__fmul_rn(dl, fmt::q3_to_float(q, 2)), __fmul_rn(dl, fmt::q3_to_float(q, 3)));
  }
}

// IQ2_S: 32 values = four groups of 8: index bytes `idx4` with their bits 8-9 in `hi` (two per group), sign bytes `sg4`,
// `sc` = two 4-bit sub-scales (first / second 16 values).
__device__ __forceinline__ void iq2s_half(float d, uint32_t idx4, uint32_t sg4, uint32_t hi, uint32_t sc, uint32_t grid_s,
                                          uint32_t (&out)[16]) {
  const float db0 = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(sc & 15u)), 0.25f);
  const float db1 = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(sc >> 4)), 0.25f);
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint32_t row = ((idx4 >> (8 * s)) & 255u) | (((hi >> (2 * s)) & 3u) << 8);
    const uint2 mag = dev::lds64(grid_s + (row << 3));
    const uint32_t sg = (sg4 >> (8 * s)) & 255u;
    const float db = s < 2 ? db0 : db1;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float m = __fmul_rn(db, fmt::byte_to_float(i < 4 ? mag.x : mag.y, i & 3));
      v[i] = __uint_as_float(__float_as_uint(m) ^ (((sg >> i) & 1u) << 31));
    }
    out[4 * s + 0] = dev::pack_bf16(v[0], v[1]);
    out[4 * s + 1] = dev::pack_bf16(v[2], v[3]);
    out[4 * s + 2] = dev::pack_bf16(v[4], v[5]);
    out[4 * s + 3] = dev::pack_bf16(v[6], v[7]);
  }
}

// Q6_K: 32 values of a 64-value slice.  `j` = which quarter of the super-block the slice is (its parity picks the low or the
// high nibbles and the bit pairs 0-3 or 4-7); `half` = first or second 32 values (nibble bytes 0-31 / 32-63, bit pair
// 2*half of the nibble-parity's four).  value = (d * scale) * (q - 32), both products exact in fp32.
__device__ __forceinline__ void q6k_half(const uint32_t (&ql)[16], const uint32_t (&qh)[8], uint32_t sc4, float d, int j, int half,
                                         uint32_t (&out)[16]) {
  const int s = j & 1;
  const uint32_t scx = sc4 ^ 0x80808080u;
  const float dsc0 = __fmul_rn(d, half ? sbyte_to_float(scx, 2) : sbyte_to_float(scx, 0));
  const float dsc1 = __fmul_rn(d, half ? sbyte_to_float(scx, 3) : sbyte_to_float(scx, 1));
  const int lo_shift = 4 * s, hi_shift = 4 * s + 2 * half;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lw = half ? ql[8 + i] : ql[i];
    const uint32_t q = ((lw >> lo_shift) & 0x0F0F0F0Fu) | (((qh[i] >> hi_shift) & 0x03030303u) << 4);
    const float dsc = i < 4 ? dsc0 : dsc1;
    out[2 * i] = dev::pack_bf16(__fmul_rn(dsc, fmt::q6_to_float(q, 0)), __fmul_rn(dsc, fmt::q6_to_float(q, 1)));
    out[2 * i + 1] = dev::pack_bf16(__fmul_rn(dsc, fmt::q6_to_float(q, 2)), __fmul_rn(dsc, fmt::q6_to_float(q, 3)));
  }
}

// What one unpack thread needs of a packed stage, held in registers: both 32-value halves of its 64-value slice of
// one W row come from the same packed bytes, so they are read from shared memory once.
//   forward: thread = one of this CTA's 128 W rows; the step selects which 64 of the row's values
//   dgrad  : thread = (W row 0..63, which 64 (`pair`, 0..3) of the 256-value column tile `ct`)
template <int QT> struct RowData;
template <> struct RowData<B2G_Q4_K> { uint4 hdr, qa, qb; };
template <> struct RowData<B2G_Q8_0> { uint32_t w[17]; };
template <> struct RowData<B2G_IQ2_XXS> { float d; uint32_t idx4[2], word[2]; };
template <> struct RowData<B2G_Q2_K> { uint32_t qs[8]; uint32_t sc4, dd; };   // 32 bytes of 2-bit values, 4 scale bytes, d | dmin
template <> struct RowData<B2G_Q3_K> { uint32_t hm[8], qs[8]; uint32_t sc_lo, sc_hi; float d; };   // mask, values, scale words
template <> struct RowData<B2G_IQ2_S> { float d; uint32_t idx[2], sg[2], hi2, sc; };   // per half: 4 index bytes, 4 sign bytes; index bits 8-9; scales
template <> struct RowData<B2G_Q5_K> { uint4 hdr, qa, qb, ha, hb; };
template <> struct RowData<B2G_Q6_K> { uint32_t ql[16], qh[8]; uint32_t sc4; float d; };   // 64 nibble bytes, 32 bit-pair bytes, 4 int8 scales

template <int QT, int MODE>
__device__ __forceinline__ void load_row(uint32_t pk, int row, int pair, int it, int ct, RowData<QT>& rd) {
  if constexpr (QT == B2G_Q4_K) {
    if constexpr (MODE == kFwd) {
      rd.hdr = dev::lds128(pk + row * 16);
      rd.qa = dev::lds128(pk + 2048 + row * 16);
      rd.qb = dev::lds128(pk + 4096 + row * 16);
    } else {
      const uint32_t r = pk + row * 144;
      rd.hdr = dev::lds128(r);
      rd.qa = dev::lds128(r + 16 + 32 * pair);
      rd.qb = dev::lds128(r + 32 + 32 * pair);
    }
  } else if constexpr (QT == B2G_Q2_K) {
    constexpr uint32_t kPiece = (MODE == kFwd ? 128u : 64u) * 16u;
    const int sb = MODE == kFwd ? (it >> 2) : ct;
    const int sft = (84 * sb) & 15;                               // 0, 4, 8 or 12
    const uint32_t base = pk + row * 16;
    uint32_t raw[12];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const uint4 v = dev::lds128(base + (2 + q) * kPiece);
      raw[4 * q] = v.x; raw[4 * q + 1] = v.y; raw[4 * q + 2] = v.z; raw[4 * q + 3] = v.w;
    }
    extract_words<8, 12>(raw, sft, rd.qs);
    const int so = sft + 4 * pair;                                 // scales[4j .. 4j+3] inside the 32-byte scale window
    rd.sc4 = dev::lds32(base + (so >> 4) * kPiece + (so & 15));
    rd.dd = dev::lds32(base + 5 * kPiece + sft);
  } else if constexpr (QT == B2G_Q3_K) {
    constexpr uint32_t kPiece = (MODE == kFwd ? 128u : 64u) * 16u;
    const int sb = MODE == kFwd ? (it >> 2) : ct;
    const int sft = (110 * sb) & 15;                              // even
    const uint32_t base = pk + row * 16;
    uint32_t raw[12];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const uint4 v = dev::lds128(base + q * kPiece);
      raw[4 * q] = v.x; raw[4 * q + 1] = v.y; raw[4 * q + 2] = v.z; raw[4 * q + 3] = v.w;
    }
    extract_words<8, 12>(raw, sft, rd.hm);
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const uint4 v = dev::lds128(base + (3 + q) * kPiece);
      raw[4 * q] = v.x; raw[4 * q + 1] = v.y; raw[4 * q + 2] = v.z; raw[4 * q + 3] = v.w;
    }
    extract_words<8, 12>(raw, sft, rd.qs);
    // scale field (12 bytes) + d (2 bytes) start `sft` bytes into the last two pieces: low nibbles of scales 4j..4j+3 in its
    // word j & 1, their high bit pairs in its word 2
    auto win = [&](int byte) { return base + (6 + (byte >> 4)) * kPiece + (byte & 15); };
    auto word_at = [&](int byte) { return dev::lds16(win(byte)) | (dev::lds16(win(byte + 2)) << 16); };
    rd.sc_lo = word_at(sft + 4 * (pair & 1));
    rd.sc_hi = word_at(sft + 8);
    rd.d = dev::half_bits_to_float(dev::lds16(win(sft + 12)));
  } else if constexpr (QT == B2G_IQ2_S) {
    // window pieces of this row; the super-block starts `sft` (even) bytes into the first; j = `pair` = quarter of the block
    constexpr uint32_t kPiece = (MODE == kFwd ? 128u : 64u) * 16u;
    const int sb = MODE == kFwd ? (it >> 2) : ct;
    const int sft = (82 * sb) & 15;
    const uint32_t base = pk + row * 16;
    auto win = [&](int byte) { return base + (byte >> 4) * kPiece + (byte & 15); };
    auto half_at = [&](int byte) { return dev::lds16(win(byte)); };
    auto word_at = [&](int byte) { return half_at(byte) | (half_at(byte + 2) << 16); };
    rd.d = dev::half_bits_to_float(half_at(sft));
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      rd.idx[half] = word_at(sft + 2 + 8 * pair + 4 * half);       // index bytes of groups 8j + 4 half .. + 3
      rd.sg[half] = word_at(sft + 34 + 8 * pair + 4 * half);       // their sign bytes
    }
    rd.hi2 = half_at(sft + 66 + 2 * pair);                         // bytes 2j, 2j+1: index bits 8-9 of four groups each
    rd.sc = half_at(sft + 74 + 2 * pair);                          // bytes 2j, 2j+1: two nibbles each, 16 values per nibble
  } else if constexpr (QT == B2G_Q5_K) {
    if constexpr (MODE == kFwd) {
      rd.hdr = dev::lds128(pk + row * 16);
      rd.ha = dev::lds128(pk + 2048 + row * 16);
      rd.hb = dev::lds128(pk + 4096 + row * 16);
      rd.qa = dev::lds128(pk + 6144 + row * 16);
      rd.qb = dev::lds128(pk + 8192 + row * 16);
    } else {
      const uint32_t r = pk + row * 176;
      rd.hdr = dev::lds128(r);
      rd.ha = dev::lds128(r + 16);
      rd.hb = dev::lds128(r + 32);
      rd.qa = dev::lds128(r + 48 + 32 * pair);
      rd.qb = dev::lds128(r + 64 + 32 * pair);
    }
  } else if constexpr (QT == B2G_Q8_0) {
    if constexpr (MODE == kFwd) load_words_shifted<17>(pk + row * 80, (68 * it) & 15, rd.w);
    else {
      const int byte0 = ((136 * (pair >> 1)) & 15) + 68 * (pair & 1);  // two blocks of column quarter `pair` inside the 144-byte window
      load_words_shifted<17>(pk + row * 144 + (byte0 & ~15), byte0 & 15, rd.w);
    }
  } else if constexpr (QT == B2G_Q6_K) {
    // pieces of this row: `piece` bytes apart, 16 bytes each; the super-block starts `sft` (even) bytes into the first line
    constexpr uint32_t kPiece = (MODE == kFwd ? 128u : 64u) * 16u;
    const int sb = MODE == kFwd ? (it >> 2) : ct;
    const int sft = (210 * sb) & 15;
    const uint32_t base = pk + row * 16;
    uint32_t raw[20];
#pragma unroll
    for (int q = 0; q < 5; ++q) {
      const uint4 v = dev::lds128(base + q * kPiece);
      raw[4 * q] = v.x; raw[4 * q + 1] = v.y; raw[4 * q + 2] = v.z; raw[4 * q + 3] = v.w;
    }
    extract_words<16, 20>(raw, sft, rd.ql);
    uint32_t rawh[12];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const uint4 v = dev::lds128(base + (5 + q) * kPiece);
      rawh[4 * q] = v.x; rawh[4 * q + 1] = v.y; rawh[4 * q + 2] = v.z; rawh[4 * q + 3] = v.w;
    }
    extract_words<8, 12>(rawh, sft, rd.qh);
    // the four scales of this 64-value slice (scales[4j .. 4j+3], j = `pair`) and d (two bytes, 16 after the scales): byte
    // offsets sft + 4j and sft + 16 into the 32-byte scale window, which lies in two pieces
    auto win = [&](int byte) { return base + (8 + (byte >> 4)) * kPiece + (byte & 15); };
    const int so = sft + 4 * pair;   // even
    const uint32_t lo = dev::lds16(win(so)), hi = dev::lds16(win(so + 2));
    rd.sc4 = lo | (hi << 16);
    rd.d = dev::half_bits_to_float(dev::lds16(win(sft + 16)));
  } else {
    // 66-byte super-block inside an 80-byte window; `off` (even) is where it starts.
    const int sb = MODE == kFwd ? (it >> 2) : ct;
    const int off = (66 * sb) & 15;
    const uint32_t h = pk + row * 80 + off;
    rd.d = dev::half_bits_to_float(dev::lds16(h));
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t q = h + 2 + 16 * pair + 8 * half;  // 8-byte group of this half (2-byte aligned)
      rd.idx4[half] = dev::lds16(q) | (dev::lds16(q + 2) << 16);
      rd.word[half] = dev::lds16(q + 4) | (dev::lds16(q + 6) << 16);
    }
  }
}

template <int QT>
__device__ __forceinline__ void decode_half(const RowData<QT>& rd, int pair, int half, uint32_t grid_s, uint32_t (&out)[16]) {
  if constexpr (QT == B2G_Q4_K) q4k_half(rd.hdr, rd.qa, rd.qb, pair, half, out);
  else if constexpr (QT == B2G_Q8_0) q8_half(rd.w, half, out);
  else if constexpr (QT == B2G_Q2_K) q2k_half(rd.qs, rd.sc4, rd.dd, pair, half, out);
  else if constexpr (QT == B2G_Q3_K) q3k_half(rd.hm, rd.qs, rd.sc_lo, rd.sc_hi, rd.d, pair, half, out);
  else if constexpr (QT == B2G_IQ2_S) iq2s_half(rd.d, rd.idx[half], rd.sg[half], (rd.hi2 >> (8 * half)) & 0xFFu, (rd.sc >> (8 * half)) & 0xFFu, grid_s, out);
  else if constexpr (QT == B2G_Q5_K) q5k_half(rd.hdr, rd.qa, rd.qb, rd.ha, rd.hb, pair, half, out);
  else if constexpr (QT == B2G_Q6_K) q6k_half(rd.ql, rd.qh, rd.sc4, rd.d, pair, half, out);
  else iq2_half(rd.d, rd.idx4[half], rd.word[half], grid_s, out);
}

__device__ __forceinline__ void st_global_v8(void* dst, const uint32_t (&w)[16], int o) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[o]), "r"(w[o + 1]), "r"(w[o + 2]), "r"(w[o + 3]),
               "r"(w[o + 4]), "r"(w[o + 5]), "r"(w[o + 6]), "r"(w[o + 7])
               : "memory");
}

// Drain one TMEM lane quarter (32 rows per row block of this CTA) of a finished tile.  A TMEM load gives each lane 32
// consecutive accumulators of ONE output row: (+ bias) -> bf16 -> two 32-byte stores, whole sectors, straight from
// registers.  This is the drain of input-gradient launches, of ragged row blocks and of short reductions; forward launches with
// long reductions take drain_block_staged below.  (Keeping the next chunk's TMEM load in flight in a second register set, and
// transposing in registers for 128-byte stores, both measured slower here.)
template <int MODE>
__device__ __forceinline__ void drain_block(const Params& p, const Tile& t, uint32_t tmem_base, int rank, int q, int lane, int m) {
  int seg = 0, col0;
  if (MODE == kFwd) { seg = t.ct / p.ct_per_seg; col0 = (t.ct - seg * p.ct_per_seg) * kBN; }
  else col0 = t.ct * kBN;
  const int ncols = MODE == kFwd ? p.n : p.k;
  __nv_bfloat16* outp = seg ? p.out1 : p.out0;
  const uint32_t acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  {
    const int row_first = m * kPairRows + rank * kBM + q * 32;
    if (row_first >= t.rows) return;             // uniform across the warp
    const bool row_ok = row_first + lane < t.rows;   // rows past a ragged expert segment belong to someone else
    __nv_bfloat16* orow = outp + static_cast<int64_t>(t.row0 + row_first + lane) * p.ldc;
#pragma unroll 1
    for (int c = 0; c < kBN / 32; ++c) {
      const int cbase = col0 + c * 32;
      if (cbase >= ncols) break;
      uint32_t r[32];
      dev::tmem_ld_32x32(acc + m * kBN + c * 32, r);
      dev::tmem_ld_wait();
      if (MODE == kFwd && p.bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (cbase + i < ncols) r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(p.bias[cbase + i]));
      }
      if (!row_ok) continue;
      __nv_bfloat16* dst = orow + cbase;
      if (p.wide_ok && cbase + 32 <= ncols) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = dev::pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        st_global_v8(dst, w, 0);
        st_global_v8(dst + 16, w, 8);
      } else {                                   // odd row pitch or the ragged last columns: element stores
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (cbase + i < ncols) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
      }
    }
  }
}

// Forward drain through shared memory: a warp whose 32 rows all belong to the tile converts 64 accumulator columns per row,
// writes them as one 128-byte row of its swizzled staging tile and lets one bulk tensor store carry the [32 x 64] box out.
// The stores of the SM then move whole 128-byte lines through the copy engine instead of one 32-byte sector per lane
// through the load/store pipe.  The staging tile is reused as soon as the previous store has READ it.
template <int MODE>
__device__ __forceinline__ void drain_block_staged(const Params& p, const Tile& t, uint32_t tmem_base, int rank, int q, int lane, int m,
                                                    uint32_t stage, const CUtensorMap* tm_o0, const CUtensorMap* tm_o1) {
  const int seg = t.ct / p.ct_per_seg, col0 = (t.ct - seg * p.ct_per_seg) * kBN;
  const CUtensorMap* om = seg ? tm_o1 : tm_o0;
  const uint32_t acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + m * kBN;
  const int row_first = m * kPairRows + rank * kBM + q * 32;
  const uint32_t srow = stage + lane * 128u, sw = static_cast<uint32_t>(lane & 7);
#pragma unroll 1
  for (int c = 0; c < kBN / 64; ++c) {
    const int cbase = col0 + c * 64;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      dev::tmem_ld_32x32(acc + c * 64 + h * 32, r);
      dev::tmem_ld_wait();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
        if (p.bias) { lo += __bfloat162float(p.bias[cbase + 32 * h + 2 * i]); hi += __bfloat162float(p.bias[cbase + 32 * h + 2 * i + 1]); }
        w[i] = dev::pack_bf16(lo, hi);
      }
      if (h == 0) {                              // the previous box must have left the staging tile
        if (lane == 0) dev::bulk_wait_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        dev::sts128(srow + ((static_cast<uint32_t>(4 * h + j) ^ sw) << 4), w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
    dev::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      dev::tma_store_2d(om, stage, cbase, t.row0 + row_first);
      dev::bulk_commit();
    }
  }
}

template <int QT, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_kernel(const Params p, const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
             const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
             const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lb,
             const __grid_constant__ CUtensorMap tm_o0, const __grid_constant__ CUtensorMap tm_o1) {
  using C = Cfg<QT, MODE>;
  using P = Packed<QT, MODE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = dev::smem_u32(smem);
  const uint32_t sA = sbase + C::kOffA, sB = sbase + C::kOffB, sP = sbase + C::kOffP;
  const uint32_t sLA = sbase + C::kOffLA, sLB = sbase + C::kOffLB;
  const uint32_t bars = sbase + C::kOffBar;
  // barrier indices.  "Full" barriers of A / B / LoRA and "accumulator empty" are used in the pair's first CTA only.
  // One `tcgen05.commit` per reduction step releases the step's A stage and B stage together (kRel + step % kRelBars): each
  // commit costs the tensor pipe about 55 cycles here (a third commit per step, to a barrier nobody waits on, measured -3.8 %).
  constexpr int kFullA = 0, kFullB = kFullA + C::kAStages, kRel = kFullB + kBStages,
                kFullP = kRel + C::kRelBars, kEmptyP = kFullP + C::kPStages, kFullL = kEmptyP + C::kPStages, kEmptyL = kFullL + 1,
                kAccFull = kEmptyL + 1, kAccEmpty = kAccFull + 1;   // kAccEmpty + m: accumulator of row block m drained
  auto bar = [&](int i) { return bars + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::kOffMisc + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = dev::cluster_ctarank();   // 0 = first CTA of the pair (issues the MMAs)
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kAStages; ++i) dev::mbar_init(bar(kFullA + i), 1);
    for (int i = 0; i < kBStages; ++i) dev::mbar_init(bar(kFullB + i), 2 * kGroupWarps);
    for (int i = 0; i < C::kRelBars; ++i) dev::mbar_init(bar(kRel + i), 1);
    for (int i = 0; i < C::kPStages; ++i) { dev::mbar_init(bar(kFullP + i), 1); dev::mbar_init(bar(kEmptyP + i), kGroupWarps * P::kSteps); }
    dev::mbar_init(bar(kFullL), 1);
    dev::mbar_init(bar(kEmptyL), 1);
    dev::mbar_init(bar(kAccFull), 1);
    dev::mbar_init(bar(kAccEmpty), 8);       // four epilogue warps in each CTA, per row block
    dev::mbar_init(bar(kAccEmpty + 1), 8);
    *abort_flag = 0;
    dev::fence_barrier_init();
    dev::fence_proxy_async_smem();
    dev::prefetch_tmap(&tm_a0);
    dev::prefetch_tmap(&tm_w0);
  }
  if constexpr (C::kGridRows > 0) {
    uint2* gs = reinterpret_cast<uint2*>(smem + C::kOffGrid);
    for (int i = threadIdx.x; i < C::kGridRows; i += kThreads) gs[i] = p.grid[i];
  }
  if (warp == 1) {
    dev::tmem_alloc_pair(dev::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    dev::tmem_relinquish_pair();
  }
  dev::tc_fence_before();
  __syncthreads();
  dev::cluster_sync_all();             // both CTAs' barriers exist before anyone signals across the pair
  dev::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_items = num_m_tiles(p) * p.num_ct;
  // first-CTA copies of the barriers that collect arrivals from both CTAs
  const uint32_t lead_full_a = dev::map_to_cta(bar(kFullA), 0), lead_full_b = dev::map_to_cta(bar(kFullB), 0);
  const uint32_t lead_full_l = dev::map_to_cta(bar(kFullL), 0), lead_acc_empty = dev::map_to_cta(bar(kAccEmpty), 0);

  if (warp == 0) {
    // ============================== TMA producer ==============================
    if (lane == 0) {
      int sa = 0, pl = 0, n = 0;                  // n: running count of reduction steps of this pair
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += num_pairs) {
        const Tile t = get_tile(p, item);
        const int nmt = t.rows > kPairRows ? 2 : 1;
        int fseg = 0, col0 = 0;
        if (MODE == kFwd) { fseg = t.ct / p.ct_per_seg; col0 = (t.ct - fseg * p.ct_per_seg) * kBN; }
        else col0 = t.ct * kBN;
        const int my_row0 = t.row0 + static_cast<int>(rank) * kBM;
        if (p.has_lora) {
          ok = dev::mbar_wait(bar(kEmptyL), pl ^ 1, abort_flag, p.status, 101);
          if (!ok) break;
          if (rank == 0) dev::mbar_arrive_expect_tx(bar(kFullL), 2 * (nmt * kLoraATile + kLoraBTile));
          for (int m = 0; m < nmt; ++m) dev::tma_load_2d_pair(sLA + m * kLoraATile, &tm_la, lead_full_l, 0, my_row0 + m * kPairRows);
          if (MODE == kFwd) {
            dev::tma_load_2d_pair(sLB, &tm_lb, lead_full_l, 0, t.expert * p.lora_rows + fseg * p.n + col0 + static_cast<int>(rank) * kBNh);
          } else {
            for (int i = 0; i < 2; ++i)
              dev::tma_load_2d_pair(sLB + i * 2048, &tm_lb, lead_full_l, col0 + static_cast<int>(rank) * kBNh + 64 * i, t.expert * 16);
          }
          pl ^= 1;
        }
        for (int it = 0; it < p.num_iters; ++it) {
          int seg = fseg, red0 = it * kBK;
          if (MODE == kDgrad) { seg = it / p.iters_per_seg; red0 = (it - seg * p.iters_per_seg) * kBK; }
          if (n >= C::kAStages) {                  // the step that used this stage last has been released
            const int r = n - C::kAStages;
            ok = dev::mbar_wait(bar(kRel + r % C::kRelBars), (r / C::kRelBars) & 1, abort_flag, p.status, 102);
            if (!ok) break;
          }
          ++n;
          if (rank == 0) dev::mbar_arrive_expect_tx(bar(kFullA + sa), 2 * nmt * kATile);   // bytes of both CTAs
          const CUtensorMap* am = (MODE == kDgrad && seg) ? &tm_a1 : &tm_a0;
          for (int m = 0; m < nmt; ++m)
            dev::tma_load_2d_pair(sA + sa * C::kAStage + m * kATile, am, lead_full_a + 8u * sa, red0, my_row0 + m * kPairRows);
          if (++sa == C::kAStages) sa = 0;
        }
      }
    }
  } else if (warp == 1) {
    // ============================== MMA issuer (first CTA of the pair) ==============================
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = dev::make_idesc_bf16(kPairRows, kBN, 0, MODE == kDgrad ? 1 : 0);
      int sa = 0, pa = 0, sb = 0, pb = 0, pl = 0, pacc = 0, n = 0;   // n: running count of reduction steps
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += num_pairs) {
        const Tile t = get_tile(p, item);
        const int nmt = t.rows > kPairRows ? 2 : 1;
        // The two row blocks of a tile have an accumulator each, and the epilogue hands them back one after the other.  The
        // next tile starts on row block 0 as soon as that one is free; the steps of row block 1 are deferred (at most
        // kMaxLag of them: every deferred step keeps its A and B stage) until the epilogue has drained it, then caught up.
        constexpr int kMaxLag = C::kAStages - 1;
        ok = dev::mbar_wait(bar(kAccEmpty), pacc ^ 1, abort_flag, p.status, 201);
        if (!ok) break;
        dev::tc_fence_after();
        bool acc1 = false;
        int pending = 0, lag_sa[kMaxLag], lag_sb[kMaxLag], lag_it[kMaxLag], lag_n[kMaxLag];
        auto issue = [&](int m, int stage_a, int stage_b, int step) {
          const uint32_t a_base = sA + stage_a * C::kAStage + m * kATile, b_base = sB + stage_b * kBStage;
#pragma unroll
          for (int k16 = 0; k16 < 4; ++k16) {
            const uint64_t bdesc = MODE == kFwd ? dev::make_smem_desc(b_base + k16 * 32, 16, 1024, 2)
                                                : dev::make_smem_desc(b_base + k16 * 2048, 8192, 1024, 2);
            const uint64_t adesc = dev::make_smem_desc(a_base + k16 * 32, 16, 1024, 2);
            dev::umma_bf16_pair(tmem_base + m * kBN, adesc, bdesc, idesc, (step | k16) != 0 ? 1u : 0u);
          }
        };
        for (int it = 0; it < p.num_iters; ++it) {
          ok = dev::mbar_wait(bar(kFullA + sa), pa, abort_flag, p.status, 202) &&
               dev::mbar_wait(bar(kFullB + sb), pb, abort_flag, p.status, 203);
          if (!ok) break;
          dev::tc_fence_after();
          if (nmt > 1 && acc1 && pending == 0) {
            // the common step: the two row blocks' MMAs alternate, so that consecutive instructions accumulate into
            // different TMEM accumulators
            const uint32_t a_base = sA + sa * C::kAStage, b_base = sB + sb * kBStage;
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
              const uint64_t bdesc = MODE == kFwd ? dev::make_smem_desc(b_base + k16 * 32, 16, 1024, 2)
                                                  : dev::make_smem_desc(b_base + k16 * 2048, 8192, 1024, 2);
#pragma unroll
              for (int m = 0; m < 2; ++m)
                dev::umma_bf16_pair(tmem_base + m * kBN, dev::make_smem_desc(a_base + m * kATile + k16 * 32, 16, 1024, 2), bdesc, idesc,
                                    (it | k16) != 0 ? 1u : 0u);
            }
            dev::umma_commit_pair(bar(kRel + n % C::kRelBars));
            ++n;
            if (++sa == C::kAStages) { sa = 0; pa ^= 1; }
            if (++sb == kBStages) { sb = 0; pb ^= 1; }
            continue;
          }
          issue(0, sa, sb, it);
          bool defer = false;
          if (!acc1) {
            if (dev::mbar_try_wait(bar(kAccEmpty + 1), pacc ^ 1)) acc1 = true;
            else if (pending < kMaxLag && it + 1 < p.num_iters) defer = true;
            else {
              ok = dev::mbar_wait(bar(kAccEmpty + 1), pacc ^ 1, abort_flag, p.status, 205);
              if (!ok) break;
              acc1 = true;
            }
            if (acc1) dev::tc_fence_after();
          }
          if (defer) {
            lag_sa[pending] = sa; lag_sb[pending] = sb; lag_it[pending] = it; lag_n[pending] = n;
            ++pending;
          } else {
            for (int d = 0; d < pending; ++d) {
              if (nmt > 1) issue(1, lag_sa[d], lag_sb[d], lag_it[d]);
              dev::umma_commit_pair(bar(kRel + lag_n[d] % C::kRelBars));
            }
            pending = 0;
            if (nmt > 1) issue(1, sa, sb, it);
            dev::umma_commit_pair(bar(kRel + n % C::kRelBars));
          }
          ++n;
          if (++sa == C::kAStages) { sa = 0; pa ^= 1; }
          if (++sb == kBStages) { sb = 0; pb ^= 1; }
        }
        if (!ok) break;
        if (p.has_lora) {
          ok = dev::mbar_wait(bar(kFullL), pl, abort_flag, p.status, 204);
          if (!ok) break;
          dev::tc_fence_after();
          const uint64_t bdesc = MODE == kFwd ? dev::make_smem_desc(sLB, 16, 256, 6) : dev::make_smem_desc(sLB, 2048, 1024, 2);
          for (int m = 0; m < nmt; ++m) {
            const uint64_t adesc = dev::make_smem_desc(sLA + m * kLoraATile, 16, 256, 6);
            dev::umma_bf16_pair(tmem_base + m * kBN, adesc, bdesc, idesc, 1u);
          }
          dev::umma_commit_pair(bar(kEmptyL));
          pl ^= 1;
        }
        dev::umma_commit_pair(bar(kAccFull));
        pacc ^= 1;
      }
    }
  } else if (warp < 6) {
    // ============================== epilogue ==============================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int pacc = 0;
    bool ok = true;
    for (int item = pair; item < total_items && ok; item += num_pairs) {
      const Tile t = get_tile(p, item);
      ok = dev::mbar_wait(bar(kAccFull), pacc, abort_flag, p.status, 301);
      if (!ok) break;
      dev::tc_fence_after();
      for (int m = 0; m < kMT; ++m) {            // a tile of one row block frees the second accumulator without reading it
        bool staged = false;
        if constexpr (C::kStaged) {
          // whole warps only: every one of the 32 rows inside the tile, every 64-column box inside the output
          const int row_first = m * kPairRows + static_cast<int>(rank) * kBM + q * 32;
          const int col_end = (t.ct % p.ct_per_seg) * kBN + kBN;
          staged = p.tma_out && row_first + 32 <= t.rows && col_end <= p.n;
          if (staged) drain_block_staged<MODE>(p, t, tmem_base, static_cast<int>(rank), q, lane, m, sbase + C::kOffStage + q * C::kStageWarp, &tm_o0, &tm_o1);
        }
        if (!staged) drain_block<MODE>(p, t, tmem_base, static_cast<int>(rank), q, lane, m);
        dev::tc_fence_before();
        __syncwarp();
        if (lane == 0) dev::mbar_arrive_cluster(lead_acc_empty + 8u * m);
      }
      pacc ^= 1;
    }
    if (C::kStaged && lane == 0) dev::bulk_wait_all();   // the staging tile must outlive the last store's read
  } else if (warp == 6 + kUnpackWarps) {
    // ============================== packed-weight producer ==============================
    if (lane == 0 && !p.hold_weights) {
      int sp = 0, pp = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += num_pairs) {
        const Tile t = get_tile(p, item);
        int fseg = 0, col0 = 0;
        if (MODE == kFwd) { fseg = t.ct / p.ct_per_seg; col0 = (t.ct - fseg * p.ct_per_seg) * kBN; }
        else col0 = t.ct * kBN;
        for (int it = 0; it < p.num_iters; ++it) {
          int seg = fseg, red0 = it * kBK;
          if (MODE == kDgrad) { seg = it / p.iters_per_seg; red0 = (it - seg * p.iters_per_seg) * kBK; }
          if (P::kSteps > 1 && (it % P::kSteps) != 0) continue;     // this step reads the slot loaded for the previous one
          ok = dev::mbar_wait(bar(kEmptyP + sp), pp ^ 1, abort_flag, p.status, 104);
          if (!ok) break;
          dev::mbar_arrive_expect_tx(bar(kFullP + sp), P::kBytes);
          const CUtensorMap* wm = seg ? &tm_w1 : &tm_w0;
          const uint32_t dst = sP + sp * C::kPStage;
          if (QT == B2G_Q6_K) {
            // ten [rows x 16 B] pieces: 5 from the line below the nibbles of half h, 3 below its bit pairs, 2 below the scales
            const int sb = MODE == kFwd ? (it >> 2) : t.ct, h = MODE == kFwd ? ((it >> 1) & 1) : static_cast<int>(rank);
            const int x0 = ((210 * sb) & ~15) >> 2;
            const int y = MODE == kFwd ? t.expert * p.n + col0 + static_cast<int>(rank) * kBNh : t.expert * p.n + red0;
            constexpr uint32_t kPiece = P::kBoxRows * 16;
            for (int q = 0; q < 5; ++q) dev::tma_load_2d(dst + q * kPiece, wm, bar(kFullP + sp), x0 + 16 * h + 4 * q, y);
            for (int q = 0; q < 3; ++q) dev::tma_load_2d(dst + (5 + q) * kPiece, wm, bar(kFullP + sp), x0 + 32 + 8 * h + 4 * q, y);
            for (int q = 0; q < 2; ++q) dev::tma_load_2d(dst + (8 + q) * kPiece, wm, bar(kFullP + sp), x0 + 48 + 4 * q, y);
          } else if (QT == B2G_Q2_K) {
            const int sb = MODE == kFwd ? (it >> 2) : t.ct, h = MODE == kFwd ? ((it >> 1) & 1) : static_cast<int>(rank);
            const int x0 = ((84 * sb) & ~15) >> 2;
            const int y = MODE == kFwd ? t.expert * p.n + col0 + static_cast<int>(rank) * kBNh : t.expert * p.n + red0;
            constexpr uint32_t kPiece = P::kBoxRows * 16;
            for (int q = 0; q < 2; ++q) dev::tma_load_2d(dst + q * kPiece, wm, bar(kFullP + sp), x0 + 4 * q, y);                  // scales
            for (int q = 0; q < 3; ++q) dev::tma_load_2d(dst + (2 + q) * kPiece, wm, bar(kFullP + sp), x0 + 4 + 8 * h + 4 * q, y);  // values of half h
            dev::tma_load_2d(dst + 5 * kPiece, wm, bar(kFullP + sp), x0 + 20, y);                                                 // d | dmin
          } else if (QT == B2G_Q3_K) {
            const int sb = MODE == kFwd ? (it >> 2) : t.ct, h = MODE == kFwd ? ((it >> 1) & 1) : static_cast<int>(rank);
            const int x0 = ((110 * sb) & ~15) >> 2;
            const int y = MODE == kFwd ? t.expert * p.n + col0 + static_cast<int>(rank) * kBNh : t.expert * p.n + red0;
            constexpr uint32_t kPiece = P::kBoxRows * 16;
            for (int q = 0; q < 3; ++q) dev::tma_load_2d(dst + q * kPiece, wm, bar(kFullP + sp), x0 + 4 * q, y);                  // mask
            for (int q = 0; q < 3; ++q) dev::tma_load_2d(dst + (3 + q) * kPiece, wm, bar(kFullP + sp), x0 + 8 + 8 * h + 4 * q, y);  // values of half h
            for (int q = 0; q < 2; ++q) dev::tma_load_2d(dst + (6 + q) * kPiece, wm, bar(kFullP + sp), x0 + 24 + 4 * q, y);       // scales, d
          } else if (QT == B2G_IQ2_S) {
            const int sb = MODE == kFwd ? (it >> 2) : t.ct;
            const int x0 = ((82 * sb) & ~15) >> 2;
            const int y = MODE == kFwd ? t.expert * p.n + col0 + static_cast<int>(rank) * kBNh : t.expert * p.n + red0;
            constexpr uint32_t kPiece = P::kBoxRows * 16;
            for (int q = 0; q < 6; ++q) dev::tma_load_2d(dst + q * kPiece, wm, bar(kFullP + sp), x0 + 4 * q, y);
          } else if (QT == B2G_Q5_K) {
            if (MODE == kFwd) {
              const int y = t.expert * p.n + col0 + static_cast<int>(rank) * kBNh;
              const int xb = 44 * (it >> 2), xq = xb + 12 + 8 * (it & 3);
              dev::tma_load_2d(dst, wm, bar(kFullP + sp), xb, y);                 // d, dmin, scales
              dev::tma_load_2d(dst + 2048, wm, bar(kFullP + sp), xb + 4, y);      // fifth bits
              dev::tma_load_2d(dst + 4096, wm, bar(kFullP + sp), xb + 8, y);
              dev::tma_load_2d(dst + 6144, wm, bar(kFullP + sp), xq, y);          // nibbles of this pair
              dev::tma_load_2d(dst + 8192, wm, bar(kFullP + sp), xq + 4, y);
            } else {
              dev::tma_load_2d(dst, wm, bar(kFullP + sp), 44 * t.ct, t.expert * p.n + red0);
            }
          } else if (MODE == kFwd) {
            const int y = t.expert * p.n + col0 + static_cast<int>(rank) * kBNh;
            if (QT == B2G_Q4_K) {
              const int xb = 36 * (it >> 2), xq = xb + 4 + 8 * (it & 3);
              dev::tma_load_2d(dst, wm, bar(kFullP + sp), xb, y);
              dev::tma_load_2d(dst + 2048, wm, bar(kFullP + sp), xq, y);
              dev::tma_load_2d(dst + 4096, wm, bar(kFullP + sp), xq + 4, y);
            } else if (QT == B2G_Q8_0) {
              dev::tma_load_2d(dst, wm, bar(kFullP + sp), ((68 * it) & ~15) >> 2, y);
            } else {
              dev::tma_load_2d(dst, wm, bar(kFullP + sp), ((66 * (it >> 2)) & ~15) >> 2, y);
            }
          } else {
            const int y = t.expert * p.n + red0;
            if (QT == B2G_Q4_K) dev::tma_load_2d(dst, wm, bar(kFullP + sp), 36 * t.ct, y);
            else if (QT == B2G_Q8_0) dev::tma_load_2d(dst, wm, bar(kFullP + sp), ((272 * t.ct + 136 * static_cast<int>(rank)) & ~15) >> 2, y);
            else dev::tma_load_2d(dst, wm, bar(kFullP + sp), ((66 * t.ct) & ~15) >> 2, y);
          }
          if (++sp == C::kPStages) { sp = 0; pp ^= 1; }
        }
      }
    }
  } else {
    // ============================== unpack ==============================
    const int tid = threadIdx.x - 6 * 32;
    const int group = tid / kGroupThreads;     // this group unpacks steps group, group + 4, group + 8, ...
    const int tg = tid % kGroupThreads;
    const uint32_t grid_s = sbase + C::kOffGrid;
    bool ok = true;
    int n = 0;                                 // running count of reduction steps of this CTA
    for (int item = pair; item < total_items && ok; item += num_pairs) {
      const int ct = item % p.num_ct;
      for (int it = 0; it < p.num_iters; ++it, ++n) {
        if ((n % kUnpackGroups) != group) continue;
        const int ps = n / P::kSteps;                                // packed slots advance once per P::kSteps steps
        const int sp = ps % C::kPStages, pp = (ps / C::kPStages) & 1;
        const int sb = n % kBStages;
        ok = dev::mbar_wait(bar(kFullP + sp), pp, abort_flag, p.status, 401, p.spin_limit);
        if (!ok) break;
        // one (row, column group) per thread: forward 128 rows, dgrad 64 rows x the two 64-column groups of this CTA
        const int drow = MODE == kFwd ? tg : (tg & 63);
        const int sub = MODE == kFwd ? 0 : (tg >> 6);                 // dgrad: which 64 of this CTA's 128 columns
        const int pairsel = MODE == kFwd ? (it & 3) : (2 * static_cast<int>(rank) + sub);   // ... of the tile's 256
        RowData<QT> rd;
        load_row<QT, MODE>(sP + sp * C::kPStage, drow, pairsel, it, ct, rd);
        const uint32_t dst = sB + sb * kBStage + static_cast<uint32_t>(sub) * 8192u + static_cast<uint32_t>(drow) * 128u;
        const uint32_t sw = static_cast<uint32_t>(drow & 7);
        // Both halves are decoded before the wait for the B slot, so that only the eight stores follow it: when the MMAs set the
        // pace, the slot comes free late and the decode is off the critical path.  IQ2_XXS forward keeps one half in registers
        // at a time: its decode is a chain of table loads, and on the short tiles of a DeepSeek expert (where the unpack warps
        // set the pace and the slot is free anyway) the second register set only costs loads in flight.
        constexpr bool kDecodeEarly = !(QT == B2G_IQ2_XXS && MODE == kFwd);
        if constexpr (kDecodeEarly) {
          uint32_t out0[16], out1[16];
          decode_half<QT>(rd, pairsel, 0, grid_s, out0);
          decode_half<QT>(rd, pairsel, 1, grid_s, out1);
          if (n >= kBStages) {                      // the step that used this slot last has been released
            const int r = n - kBStages;
            ok = dev::mbar_wait(bar(kRel + r % C::kRelBars), (r / C::kRelBars) & 1, abort_flag, p.status, 402);
            if (!ok) break;
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            dev::sts128(dst + ((static_cast<uint32_t>(c) ^ sw) << 4), out0[4 * c], out0[4 * c + 1], out0[4 * c + 2], out0[4 * c + 3]);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            dev::sts128(dst + ((static_cast<uint32_t>(4 + c) ^ sw) << 4), out1[4 * c], out1[4 * c + 1], out1[4 * c + 2], out1[4 * c + 3]);
        } else {
          if (n >= kBStages) {                      // the step that used this slot last has been released
            const int r = n - kBStages;
            ok = dev::mbar_wait(bar(kRel + r % C::kRelBars), (r / C::kRelBars) & 1, abort_flag, p.status, 402);
            if (!ok) break;
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t out[16];
            decode_half<QT>(rd, pairsel, half, grid_s, out);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              dev::sts128(dst + ((static_cast<uint32_t>(4 * half + c) ^ sw) << 4), out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
          }
        }
        dev::fence_proxy_async_smem();
        __syncwarp();
        // The proxy fence above also covers the packed slot: its bytes were read through the generic proxy and the refill
        // is a TMA (async proxy) write.  Handing the slot back right after the loads, without a fence in between, let the
        // refill overtake the reads.
        if (lane == 0) {
          dev::mbar_arrive(bar(kEmptyP + sp));
          dev::mbar_arrive_cluster(lead_full_b + 8u * sb);
        }
      }
    }
  }

  // Neither CTA may leave (or free TMEM) while its partner can still signal it or read its shared memory.
  dev::tc_fence_before();
  __syncthreads();
  dev::cluster_sync_all();
  if (warp == 1) {
    dev::tc_fence_after();
    dev::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
struct Launch {
  int qtype, mode;
  int padded;                 // payload rows are padded to the next multiple of 16 bytes (B2G_PADDED_ROWS flag of the type id)
  const void *a0, *a1;        // activations [m_total, red_dim]
  const void *w0, *w1;        // payloads
  const void *la, *lb;        // LoRA operands
  int64_t m_total, n, k;
  int64_t lda, ldc;           // row pitch (elements) of the activation operand / the output; 0 = contiguous
  int num_experts;
  const int32_t* tiles;       // nullptr = dense
  int64_t lora_rows;
  void *out0, *out1;
  const void* bias;
  int* status;
  cudaStream_t stream;
  uint32_t spin_limit;        // 0 = the library's default
  int hold_weights;           // test hook, see Params
};

// Row pitch of a payload: the format's bytes per row, or that rounded up to 16 when the caller padded the rows.
inline int64_t packed_pitch(int qtype, int64_t k, int padded) {
  const int64_t b = fmt::row_bytes(qtype, k);
  return padded ? (b + 15) / 16 * 16 : b;
}
// The `qtype` argument of the entry points: GGML type id, optionally with B2G_PADDED_ROWS.
inline void split_qtype(int arg, Launch& L) {
  L.qtype = arg & 0xFF;
  L.padded = (arg & B2G_PADDED_ROWS) ? 1 : 0;
}

template <int QT, int MODE>
int launch_impl(const Launch& L) {
  using C = Cfg<QT, MODE>;
  using P = Packed<QT, MODE>;
  Params p{};
  p.m_total = (int)L.m_total; p.n = (int)L.n; p.k = (int)L.k;
  p.nseg = L.w1 ? 2 : 1;
  const int red_cols = MODE == kFwd ? p.k : p.n;  // width of the activation operand
  if (MODE == kFwd) {
    p.ct_per_seg = (p.n + kBN - 1) / kBN;
    p.num_ct = p.nseg * p.ct_per_seg;
    p.num_iters = p.k / kBK;
    p.iters_per_seg = p.num_iters;
    p.ldc = L.ldc ? (int)L.ldc : p.n;
  } else {
    p.ct_per_seg = p.k / kBN;
    p.num_ct = p.k / kBN;
    p.iters_per_seg = (p.n + kBK - 1) / kBK;
    p.num_iters = p.nseg * p.iters_per_seg;
    p.ldc = L.ldc ? (int)L.ldc : p.k;
  }
  p.dense_m_tiles = (int)((L.m_total + kTileRows - 1) / kTileRows);
  p.has_lora = L.la != nullptr;
  p.lora_rows = (int)L.lora_rows;
  p.tiles = reinterpret_cast<const int4*>(L.tiles);
  p.out0 = static_cast<__nv_bfloat16*>(L.out0);
  p.out1 = static_cast<__nv_bfloat16*>(L.out1);
  p.bias = static_cast<const __nv_bfloat16*>(L.bias);
  p.status = L.status;
  p.spin_limit = L.spin_limit ? L.spin_limit : B2G_SPIN_LIMIT;
  p.hold_weights = L.hold_weights;
  p.wide_ok = (p.ldc % 16 == 0) && (reinterpret_cast<uintptr_t>(L.out0) % 32 == 0) && (reinterpret_cast<uintptr_t>(L.out1) % 32 == 0);
  p.grid = nullptr;
  if (QT == B2G_IQ2_S) {
    int rc = iq2s_grid(&p.grid);
    if (rc) return rc;
  }
  if (QT == B2G_IQ2_XXS) {
    int rc = iq2xxs_grid(&p.grid);
    if (rc) return rc;
  }

  // First a runtime call: it binds the device's primary context to this thread.  The tensor-map encoder below is a driver
  // entry point and fails with CUDA_ERROR_INVALID_CONTEXT on a thread that has made no runtime call yet (an autograd
  // worker whose first CUDA work is this launch).
  auto kern = qgemm_kernel<QT, MODE>;
  B2G_KERNEL_SMEM(kern, C::kSmemBytes);
  CUtensorMap tm_a0, tm_a1, tm_w0, tm_w1, tm_la, tm_lb;
  int rc;
  const uint64_t a_pitch = (uint64_t)(L.lda ? L.lda : red_cols) * 2;
  if ((rc = make_tmap_2d(&tm_a0, L.a0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, red_cols, L.m_total, a_pitch, kBK, kBM,
                         CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  tm_a1 = tm_a0;
  if (L.a1 && (rc = make_tmap_2d(&tm_a1, L.a1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, red_cols, L.m_total, a_pitch, kBK, kBM,
                                 CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  const uint64_t w_pitch = (uint64_t)packed_pitch(QT, L.k, L.padded);
  const uint64_t w_rows = (uint64_t)L.num_experts * L.n;
  if ((rc = make_tmap_2d(&tm_w0, L.w0, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w_pitch / 4, w_rows, w_pitch, P::kBoxWords, P::kBoxRows,
                         CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  tm_w1 = tm_w0;
  if (L.w1 && (rc = make_tmap_2d(&tm_w1, L.w1, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w_pitch / 4, w_rows, w_pitch, P::kBoxWords,
                                 P::kBoxRows, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  tm_la = tm_a0; tm_lb = tm_a0;
  if (p.has_lora) {
    if ((rc = make_tmap_2d(&tm_la, L.la, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 16, L.m_total, 32, 16, kBM,
                           CU_TENSOR_MAP_SWIZZLE_32B))) return rc;
    if (MODE == kFwd) {
      if ((rc = make_tmap_2d(&tm_lb, L.lb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 16, (uint64_t)L.num_experts * L.lora_rows, 32, 16,
                             kBNh, CU_TENSOR_MAP_SWIZZLE_32B))) return rc;
    } else {
      if ((rc = make_tmap_2d(&tm_lb, L.lb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, L.k, (uint64_t)L.num_experts * 16, (uint64_t)L.k * 2,
                             64, 16, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    }
  }

  // Staged drain (forward, types whose packed slots leave 16 KB of shared memory): worth it when the reduction is long enough
  // for the drain to run beside the next tile's MMAs and the unpack warps' shared-memory traffic (measured: +4 % at 32 steps
  // per tile, -3 % at 8, where nothing else is in the load/store pipe and the wait for the staging tile shows).
  CUtensorMap tm_o0 = tm_a0, tm_o1 = tm_a0;
  p.tma_out = 0;
  if (C::kStaged && p.wide_ok && L.n % 8 == 0 && p.num_iters >= 16) {
    const uint64_t o_pitch = (uint64_t)p.ldc * 2;
    if ((rc = make_tmap_2d(&tm_o0, L.out0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, L.n, L.m_total, o_pitch, 64, 32,
                           CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    tm_o1 = tm_o0;
    if (L.out1 && (rc = make_tmap_2d(&tm_o1, L.out1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, L.n, L.m_total, o_pitch, 64, 32,
                                     CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    p.tma_out = 1;
  }

  int pairs = (sm_count() - gemm_sm_margin()) / 2;
  if (pairs < 1) pairs = 1;
  if (!L.tiles) {
    const int64_t items = (int64_t)p.dense_m_tiles * p.num_ct;
    if (items < pairs) pairs = (int)items;
  }
  if (pairs < 1) return 0;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = L.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B2G_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p, tm_a0, tm_a1, tm_w0, tm_w1, tm_la, tm_lb, tm_o0, tm_o1));
  return 0;
}

template <int MODE>
int launch_mode(const Launch& L) {
  switch (L.qtype) {
    case B2G_Q4_K: return launch_impl<B2G_Q4_K, MODE>(L);
    case B2G_Q8_0: return launch_impl<B2G_Q8_0, MODE>(L);
    case B2G_IQ2_XXS: return launch_impl<B2G_IQ2_XXS, MODE>(L);
    case B2G_Q2_K: return launch_impl<B2G_Q2_K, MODE>(L);
    case B2G_Q3_K: return launch_impl<B2G_Q3_K, MODE>(L);
    case B2G_IQ2_S: return launch_impl<B2G_IQ2_S, MODE>(L);
    case B2G_Q5_K: return launch_impl<B2G_Q5_K, MODE>(L);
    case B2G_Q6_K: return launch_impl<B2G_Q6_K, MODE>(L);
    default: return fail(B2G_E_ARG, "unsupported GGUF type id %d (supported: 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K, 13 Q5_K, 14 Q6_K, 16 IQ2_XXS, 22 IQ2_S)", L.qtype);
  }
}

int check_common(const Launch& L, const char* what) {
  B2G_REQUIRE(L.m_total >= 0 && L.n > 0 && L.k > 0, "%s: bad shape M=%lld N=%lld K=%lld", what, (long long)L.m_total,
              (long long)L.n, (long long)L.k);
  B2G_REQUIRE(L.k % 256 == 0, "%s: K=%lld must be a multiple of 256", what, (long long)L.k);
  B2G_REQUIRE(packed_pitch(L.qtype, L.k, L.padded) % 16 == 0,
              "%s: packed rows of %lld bytes are not 16-byte multiples: pad every row to the next multiple of 16 bytes and pass the type "
              "id with B2G_PADDED_ROWS", what, (long long)fmt::row_bytes(L.qtype, L.k));
  B2G_REQUIRE(L.m_total < (1ll << 31) && (int64_t)L.num_experts * L.n < (1ll << 31), "%s: shape too large", what);
  B2G_REQUIRE(L.m_total == 0 || (L.a0 && L.w0 && L.out0), "%s: null pointer", what);
  B2G_REQUIRE((L.la == nullptr) == (L.lb == nullptr), "%s: the two LoRA operands come together", what);
  return 0;
}

// ---- grouped tile table ------------------------------------------------------------------------
// Offsets are clamped to [0, total_rows] and kept monotone, and no more entries are written than the table holds, so that a
// caller whose offsets overrun the activation matrix (an expert-parallel receive buffer that was too small) gets tiles that
// stay inside it; status 904 reports the overrun.
// Tiles that fill both row blocks come first, the ragged ends of at most one row block (half the MMAs, about half the time)
// after them, each class in expert order: CTA pairs take table entries round-robin, so every pair gets the same number of
// tiles of each class to within one, which an order by expert alone does not give (experts of about one tile of rows
// alternate long and short entries, and the period of that pattern beats against the number of pairs).
__global__ void __launch_bounds__(256) schedule_kernel(const int64_t* __restrict__ expert_indices, const int32_t* __restrict__ offsets,
                                                       const int32_t* __restrict__ first_row, int G, int rows_per_tile, int total_rows,
                                                       int max_tiles, int4* __restrict__ tiles, int* __restrict__ status) {
  __shared__ int scan_tall[256], scan_short[256];
  __shared__ int carry_tall, carry_short, total_tall;
  const int half_tile = rows_per_tile / 2;
  auto segment = [&](int g, int& begin, int& rows) {
    begin = 0; rows = 0;
    if (g >= G) return;
    begin = g > 0 ? offsets[g - 1] : (first_row ? *first_row : 0);
    int end = offsets[g];
    if (end > total_rows || begin > total_rows) {
      if (status) atomicCAS(status, 0, 904);
      end = end > total_rows ? total_rows : end;
      begin = begin > total_rows ? total_rows : begin;
    }
    if (begin < 0) begin = 0;
    rows = end - begin;
    if (rows < 0) rows = 0;
  };
  // pass 1: how many tiles fill both row blocks
  int mine = 0;
  for (int g = threadIdx.x; g < G; g += 256) {
    int begin, rows;
    segment(g, begin, rows);
    const int nt = (rows + rows_per_tile - 1) / rows_per_tile;
    const int last = rows - (nt - 1) * rows_per_tile;
    mine += nt - (nt > 0 && last <= half_tile ? 1 : 0);
  }
  scan_tall[threadIdx.x] = mine;
  if (threadIdx.x == 0) { carry_tall = 0; carry_short = 0; }
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) scan_tall[threadIdx.x] += scan_tall[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) total_tall = scan_tall[0];
  __syncthreads();
  // pass 2: place them
  for (int g0 = 0; g0 < G; g0 += 256) {
    const int g = g0 + threadIdx.x;
    int begin, rows;
    segment(g, begin, rows);
    const int nt = (rows + rows_per_tile - 1) / rows_per_tile;
    const int last = rows - (nt - 1) * rows_per_tile;
    const int n_short = nt > 0 && last <= half_tile ? 1 : 0, n_tall = nt - n_short;
    scan_tall[threadIdx.x] = n_tall;
    scan_short[threadIdx.x] = n_short;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
      const int add_t = threadIdx.x >= off ? scan_tall[threadIdx.x - off] : 0;
      const int add_s = threadIdx.x >= off ? scan_short[threadIdx.x - off] : 0;
      __syncthreads();
      scan_tall[threadIdx.x] += add_t;
      scan_short[threadIdx.x] += add_s;
      __syncthreads();
    }
    if (g < G) {
      const int e = static_cast<int>(expert_indices[g]);
      const int first_tall = carry_tall + scan_tall[threadIdx.x] - n_tall;
      for (int i = 0; i < n_tall && first_tall + i < max_tiles; ++i) {
        const int left = rows - i * rows_per_tile;
        tiles[1 + first_tall + i] = make_int4(e, begin + i * rows_per_tile, left < rows_per_tile ? left : rows_per_tile, g);
      }
      const int at = total_tall + carry_short + scan_short[threadIdx.x] - n_short;
      if (n_short && at < max_tiles) tiles[1 + at] = make_int4(e, begin + (nt - 1) * rows_per_tile, last, g);
    }
    __syncthreads();
    if (threadIdx.x == 255) { carry_tall += scan_tall[255]; carry_short += scan_short[255]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const int total = total_tall + carry_short;
    tiles[0] = make_int4(total < max_tiles ? total : max_tiles, rows_per_tile, G, 0);
  }
}

}  // namespace qg
}  // namespace b2g

using namespace b2g;

extern "C" int b2g_qlinear_fwd(int qtype, const void* x, const void* payload, const void* bias, const void* xas, const void* lora_b16,
                               void* y, int64_t M, int64_t N, int64_t K, int* status, void* stream) {
  qg::Launch L{};
  qg::split_qtype(qtype, L); L.mode = qg::kFwd; L.a0 = x; L.w0 = payload; L.la = xas; L.lb = lora_b16;
  L.m_total = M; L.n = N; L.k = K; L.num_experts = 1; L.lora_rows = N; L.out0 = y; L.bias = bias; L.status = status;
  L.stream = static_cast<cudaStream_t>(stream);
  int rc = qg::check_common(L, "qlinear_fwd");
  if (rc) return rc;
  if (M == 0) return 0;
  return qg::launch_mode<qg::kFwd>(L);
}

// Test hook for the bounded waits: the forward product with its packed-weight producer held back and a short wait limit.  The
// unpack warps' wait for packed bytes (site 401) runs out after `spin_limit` polls, the CTA's abort flag stops every other role
// (their own waits poll that flag),
// TMEM is freed and the kernel returns with *status = 401 and an unspecified Y.  Nothing faults, traps or hangs; the next launch
// on the same stream is unaffected.
extern "C" int b2g_debug_stalled_qlinear_fwd(int qtype, const void* x, const void* payload, void* y, int64_t M, int64_t N, int64_t K,
                                             int spin_limit, int* status, void* stream) {
  qg::Launch L{};
  qg::split_qtype(qtype, L); L.mode = qg::kFwd; L.a0 = x; L.w0 = payload;
  L.m_total = M; L.n = N; L.k = K; L.num_experts = 1; L.lora_rows = N; L.out0 = y; L.status = status;
  L.stream = static_cast<cudaStream_t>(stream);
  L.spin_limit = static_cast<uint32_t>(spin_limit); L.hold_weights = 1;
  B2G_REQUIRE(spin_limit >= 16 && spin_limit <= (1 << 16), "debug_stalled_qlinear_fwd: spin limit %d outside 16..65536", spin_limit);
  B2G_REQUIRE(status != nullptr, "debug_stalled_qlinear_fwd: a status word is required");
  int rc = qg::check_common(L, "debug_stalled_qlinear_fwd");
  if (rc) return rc;
  if (M == 0) return 0;
  return qg::launch_mode<qg::kFwd>(L);
}

extern "C" int b2g_qlinear_dgrad(int qtype, const void* dy, const void* payload, const void* dybs, const void* lora_a16, void* dx,
                                 int64_t M, int64_t N, int64_t K, int* status, void* stream) {
  qg::Launch L{};
  qg::split_qtype(qtype, L); L.mode = qg::kDgrad; L.a0 = dy; L.w0 = payload; L.la = dybs; L.lb = lora_a16;
  L.m_total = M; L.n = N; L.k = K; L.num_experts = 1; L.lora_rows = 16; L.out0 = dx; L.status = status;
  L.stream = static_cast<cudaStream_t>(stream);
  int rc = qg::check_common(L, "qlinear_dgrad");
  if (rc) return rc;
  B2G_REQUIRE(N % 8 == 0, "qlinear_dgrad: N=%lld must be a multiple of 8 (pad dY)", (long long)N);
  if (M == 0) return 0;
  return qg::launch_mode<qg::kDgrad>(L);
}

static int64_t grouped_max_tiles(int64_t R, int G) { return R / qg::kTileRows + G + 1; }   // every expert may end in one partial tile

extern "C" int64_t b2g_grouped_tiles_bytes(int64_t R, int G) { return (1 + grouped_max_tiles(R, G)) * (int64_t)sizeof(int4); }

extern "C" int b2g_grouped_schedule(const int64_t* expert_indices, const int32_t* offsets, const int32_t* first_row, int G, int64_t R,
                                    int32_t* tiles, int* status, void* stream) {
  B2G_REQUIRE(G >= 0 && R >= 0 && R < (1ll << 31) && tiles, "bad arguments");
  B2G_REQUIRE(aligned16(tiles), "tile table must be 16-byte aligned");
  B2G_REQUIRE(G == 0 || (expert_indices && offsets), "null pointer");
  B2G_KERNEL_MAX_SHARED(qg::schedule_kernel);
  qg::schedule_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(expert_indices, offsets, first_row, G, qg::kTileRows,
                                                                       (int)R, (int)grouped_max_tiles(R, G),
                                                                       reinterpret_cast<int4*>(tiles), status);
  B2G_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int b2g_grouped_fwd(int qtype, const void* x, const void* payload0, const void* payload1, const int32_t* tiles,
                               const void* xas, const void* lora_b16, int64_t lora_rows, void* y0, void* y1, int64_t R, int64_t N,
                               int64_t K, int num_experts, int* status, void* stream) {
  qg::Launch L{};
  qg::split_qtype(qtype, L); L.mode = qg::kFwd; L.a0 = x; L.w0 = payload0; L.w1 = payload1; L.la = xas; L.lb = lora_b16;
  L.m_total = R; L.n = N; L.k = K; L.num_experts = num_experts; L.tiles = tiles; L.lora_rows = lora_rows;
  L.out0 = y0; L.out1 = y1; L.status = status; L.stream = static_cast<cudaStream_t>(stream);
  int rc = qg::check_common(L, "grouped_fwd");
  if (rc) return rc;
  B2G_REQUIRE(tiles && num_experts >= 1, "grouped_fwd: tile table missing");
  B2G_REQUIRE((payload1 == nullptr) == (y1 == nullptr), "grouped_fwd: second payload and second output come together");
  B2G_REQUIRE(N % 8 == 0, "grouped_fwd: N=%lld must be a multiple of 8", (long long)N);
  if (R == 0) return 0;
  return qg::launch_mode<qg::kFwd>(L);
}

extern "C" int b2g_grouped_dgrad(int qtype, const void* dy0, const void* dy1, const void* payload0, const void* payload1,
                                 const int32_t* tiles, const void* dybs, const void* lora_a16, void* dx, int64_t R, int64_t N,
                                 int64_t K, int num_experts, int* status, void* stream) {
  qg::Launch L{};
  qg::split_qtype(qtype, L); L.mode = qg::kDgrad; L.a0 = dy0; L.a1 = dy1; L.w0 = payload0; L.w1 = payload1; L.la = dybs; L.lb = lora_a16;
  L.m_total = R; L.n = N; L.k = K; L.num_experts = num_experts; L.tiles = tiles; L.lora_rows = 16;
  L.out0 = dx; L.status = status; L.stream = static_cast<cudaStream_t>(stream);
  int rc = qg::check_common(L, "grouped_dgrad");
  if (rc) return rc;
  B2G_REQUIRE(tiles && num_experts >= 1, "grouped_dgrad: tile table missing");
  B2G_REQUIRE((payload1 == nullptr) == (dy1 == nullptr), "grouped_dgrad: second payload and second gradient come together");
  B2G_REQUIRE(N % 64 == 0, "grouped_dgrad: N=%lld must be a multiple of 64", (long long)N);
  if (R == 0) return 0;
  return qg::launch_mode<qg::kDgrad>(L);
}

// ---- fixed groups: G independent dense products on column blocks of one activation tensor ----------------------
static int fixed_grouped(int mode, int qtype, const void* a, const void* payload, void* out, int64_t M, int groups, int64_t N, int64_t K,
                         int* status, void* stream, const char* what) {
  B2G_REQUIRE(groups >= 1 && groups <= 64, "%s: group count %d outside 1..64", what, groups);
  const int64_t in_w = mode == qg::kFwd ? K : N, out_w = mode == qg::kFwd ? N : K;
  B2G_REQUIRE(in_w % 8 == 0 && out_w % 16 == 0, "%s: group widths %lld -> %lld must be multiples of 8 / 16", what, (long long)in_w,
              (long long)out_w);
  const int64_t row_bytes = qg::packed_pitch(qtype & 0xFF, K, (qtype & B2G_PADDED_ROWS) ? 1 : 0);
  for (int g = 0; g < groups; ++g) {
    qg::Launch L{};
    qg::split_qtype(qtype, L); L.mode = mode;
    L.a0 = static_cast<const __nv_bfloat16*>(a) + g * in_w;
    L.w0 = static_cast<const uint8_t*>(payload) + (int64_t)g * N * row_bytes;
    L.out0 = static_cast<__nv_bfloat16*>(out) + g * out_w;
    L.lda = groups * in_w; L.ldc = groups * out_w;
    L.m_total = M; L.n = N; L.k = K; L.num_experts = 1; L.lora_rows = mode == qg::kFwd ? N : 16; L.status = status;
    L.stream = static_cast<cudaStream_t>(stream);
    int rc = qg::check_common(L, what);
    if (rc) return rc;
    if (M == 0) return 0;
    rc = mode == qg::kFwd ? qg::launch_mode<qg::kFwd>(L) : qg::launch_mode<qg::kDgrad>(L);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int b2g_fixed_grouped_fwd(int qtype, const void* x, const void* payload, void* y, int64_t M, int groups, int64_t N, int64_t K,
                                     int* status, void* stream) {
  return fixed_grouped(qg::kFwd, qtype, x, payload, y, M, groups, N, K, status, stream, "fixed_grouped_fwd");
}

extern "C" int b2g_fixed_grouped_dgrad(int qtype, const void* dy, const void* payload, void* dx, int64_t M, int groups, int64_t N,
                                       int64_t K, int* status, void* stream) {
  B2G_REQUIRE(N % 8 == 0, "fixed_grouped_dgrad: N=%lld must be a multiple of 8", (long long)N);
  return fixed_grouped(qg::kDgrad, qtype, dy, payload, dx, M, groups, N, K, status, stream, "fixed_grouped_dgrad");
}
