// Decode path for 1 <= M <= 8 rows of a large matrix on the integer tensor-core path (tcgen05.mma kind::i8):
// the packed nibbles reach the tensor core with ONE logic operation per packed word, no conversion to floating
// point at all, and half of them with no operation.
//
// A byte of the packed weights holds two nibbles of one column, q_hi (bits 4..7) and q_lo (bits 0..3), for two
// different k of the same 128-k block.  Two unsigned 8-bit operands are used:
//     raw = the packed bytes as the copy engine left them in shared memory (16 * q_hi + q_lo),
//     hi  = word & 0xf0f0f0f0 (bytes 16 * q_hi), written to tensor memory (lane = output column, one byte per slot).
// The activations of a block are turned into block-fixed-point integers once per unit by two helper warps:
//     x[m, k] ~ sx[m] * t[m, k],   t = rint(x / sx) in [-16256, 16256],   sx = max_k |x[m, k]| / 16256
//     t = 128 * p1 + p2,  p1 in [-127, 127], p2 in [-64, 63]                  (two signed 8-bit planes)
// and laid out as the B operand, the k slots in the order of the bytes they meet: tile Xhi (rows 0..7) for the k of
// the high nibbles, tile Xlo (rows 8..15, directly behind) for the k of the low nibbles; plane 1 of row m in row m
// of a tile, plane 2 in row MR + m.  One MMA of N = 16 over [Xhi; Xlo] and one over Xlo give (int32, exact)
//     D_hi[n, 0..7]  = sum_slots hi * Xhi      D_hi[n, 8..15] = sum_slots hi * Xlo      D_raw[n, 0..7] = sum_slots raw * Xlo
// and, since raw - hi = q_lo byte by byte, D_raw - D_hi[8..] = sum_slots q_lo * Xlo:
//     y[m, n] += s[n] * sx[m] * ( (128 * D_hi[m] + D_hi[MR + m]) / 16
//                                 + 128 * (D_raw[m] - D_hi[8 + m]) + (D_raw[MR + m] - D_hi[8 + MR + m]) - z[n] * T[m] )
// with T[m] = sum_k t[m, k]; everything inside the parenthesis is exact integer arithmetic, so the only
// roundings are the quantisation of x (15 bits below the largest activation of the row's 128-k block, i.e.
// finer than the fp16 spacing of that activation) and one fp32 multiply-add per unit.  Like the reference's
// GEMV (LLMQRT/runtime_refact/csrc/awq/gemv.cu:138) the weights are applied un-rounded, s * (q - z).
//
// Work distribution is the split-K stream of the exact-weight kernel (awq_skinny.cu): unit = 256 columns x 128 k
// (16 KiB of packed weights), CTA b owns units [b*U/G, (b+1)*U/G) of the flattened (column tile, k block)
// sequence, one copy pipeline per CTA that never drains; a column tile that straddles CTAs is finished through
// fp32 partials added in CTA (= k) order by the last contributor.  Deterministic; a row's bits do not depend on M.
//
// TWO CTAs per SM (384 threads, 256 tensor-memory columns, ~100 KB of shared memory each).  With two small CTAs
// per SM the next kernel of the stream (programmatic dependent launch) takes over an SM half as soon as one CTA
// has left, and its first copies overlap the other CTA's tail.
//
// Warps: 0 copy producer, 1 MMA issuer, 2..9 two groups of four warps that mask the words into tensor memory
// (a thread serves one column in each 128-column half) and fold the finished accumulators, 10..11 activation
// helpers (alternate units).  TMEM columns: [0, 128) two accumulator windows of 64 (2 halves x {hi, raw} x 16),
// [128, 256) two operand slots of 64 (2 halves x 32, of which the hi bytes take 16 columns = 64 k slots).  Per
// unit the tensor core runs 8 instructions (2 halves x 2 k steps of 32 slots x {hi, raw}).  A group folds unit u
// when it starts on unit u + 2.  Every mbarrier wait is bounded (see awq_ptx.cuh).
//
// 5..8 rows (MR = 8): the activation tiles have 16 rows (plane 1 of row m in tile row 2 m, plane 2 in 2 m + 1), the
// hi MMA has N = 32 over [Xhi; Xlo] and the raw MMA N = 16 over Xlo; accumulator windows of 96 columns
// (2 halves x {hi 32, raw 16}) at [0, 192), operand slots of 32 columns at [192, 256); stages of 19 KiB.
//
// Who builds the activation planes.  Up to 2 rows: the two helper warps of every CTA, for each of its units.  That
// work is the same in every CTA that meets a k block (a 70B gate_up has 14,336 units and 64 k blocks), it grows
// with the rows, and its latency (two shuffle reductions, a division, conversions: ~1 us per pair of rows and
// unit) bounds the kernel from 3 rows on (measured on 8192 -> 57344 with the helpers' arithmetic taken out:
// 4 rows 53 -> 48 us, 8 rows 89 -> 63 us).  From 3 rows (PREP kernels) d8_prep_kernel writes the planes and
// (sx, T) of every k block once per call into the workspace, the copy producer fetches a unit's record with its
// weights (two more bulk copies per unit) and the CTAs have no helper warps (320 threads): 4 rows 53.9 -> 50.7 us,
// 8 rows 58.4 us (exact-weight kernel: 75 us).  At 1 and 2 rows the second launch costs more than it saves
// (45.1 -> 45.7, 45.2 -> 47.0 us).  The bits are the same either way.
#include "awq_gemv_common.cuh"
#include "awq_peer.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kD8UnpackWarps = 8;
constexpr int kD8UnpackThreads = kD8UnpackWarps * 32;
constexpr int kD8Groups = 2;
constexpr int kD8HelperWarps = 2;
constexpr int kD8Threads = 64 + kD8UnpackThreads + kD8HelperWarps * 32;   // 12 warps
constexpr int kD8HelperWarp0 = 2 + kD8UnpackWarps;
constexpr int kD8CtasPerSm = 2;
constexpr int kD8BN = 256;
constexpr int kD8RawBytes = kD8BN * 64;            // [256 columns][64 bytes], 64-byte swizzle
constexpr int kD8RawOff = 0;
constexpr int kD8XhiOff = kD8RawOff + kD8RawBytes;
constexpr int kD8Windows = 2;
constexpr int kD8AStages = 2;
constexpr int kD8TmemCols = 256;
constexpr int kD8MetaSlots = 8;                    // ring of per-unit (sx, T) rows (see the helpers for why 8 is enough)
constexpr int kD8MaxRows = 8;                      // beyond that the per-row fold costs more than the exact-weight kernel's unpack
constexpr int kD8Range = 16256;                    // 127 * 128: largest |t|

template <int MR> struct D8Cfg {
  static_assert(MR == 1 || MR == 2 || MR == 4 || MR == 8, "rows per call class");
  // B operand tiles: kXRows rows x 64 k slots, 64-byte swizzle (8-row groups of 512 bytes).  Up to four rows: only
  // tile rows 0 .. 2 MR - 1 <= 7 carry data (plane 1 of row m in row m, plane 2 in row MR + m) and a tile takes 512
  // bytes; the instructions have N = 16 and also read the 8 rows behind the tile they start at, whose products
  // land in accumulator columns nobody looks at.  Eight rows: 16-row tiles, plane 1 of row m in row 2 m, plane 2
  // in row 2 m + 1; the hi MMA has N = 32.
  static constexpr int kXRows = MR == 8 ? 16 : 8;
  static constexpr int kXTileBytes = kXRows * 64;
  static constexpr int kXloOff = kD8XhiOff + kXTileBytes;
  static constexpr int kSzOff = kXloOff + kXTileBytes;       // 256 fp16 scales, then 32 qzeros words
  static constexpr int kStageBytes = MR == 8 ? 19 * 1024 : 18 * 1024;
  static constexpr int kHiN = MR == 8 ? 32 : 16;             // N of the MMA over [Xhi; Xlo]
  static constexpr int kHalfCols = kHiN + 16;                // accumulator columns of a 128-column half: hi, then raw (N = 16)
  static constexpr int kWinCols = 2 * kHalfCols;             // 64 / 96
  static constexpr int kABase = kD8Windows * kWinCols;       // 128 / 192
  static constexpr int kASlot = MR == 8 ? 32 : 64;           // operand slot; a half's 16 columns start at h * kASlot / 2
  static_assert(kSzOff + 512 + 128 <= kStageBytes && kStageBytes % 1024 == 0, "stage layout");
  static_assert(kXloOff + 1024 <= kStageBytes, "the rows the tensor core reads behind a tile stay inside the stage");
  static_assert(kABase + kD8AStages * kASlot == kD8TmemCols, "tensor memory columns");
  __host__ __device__ static constexpr int plane1_row(int m) { return MR == 8 ? 2 * m : m; }
  __host__ __device__ static constexpr int plane2_row(int m) { return MR == 8 ? 2 * m + 1 : MR + m; }
  // Record of one k block as d8_prep_kernel writes it: tile Xhi, tile Xlo, MR x (sx bits, T).
  static constexpr int kPrepMetaBytes = MR * 8 < 16 ? 16 : MR * 8;
  static constexpr int kPrepRecBytes = 2 * kXTileBytes + kPrepMetaBytes;
  static constexpr int kMetaStride = kPrepMetaBytes / 8;     // int2 entries per ring slot
  static constexpr int kCombBytes = (kD8Groups - 1) * kD8BN * MR * 4;
  static constexpr int kMetaBytes = kD8MetaSlots * kPrepMetaBytes;
  static constexpr int kStages = 5;                          // per CTA; two CTAs per SM (six measured no faster)
  static constexpr int kCombOff = kStages * kStageBytes;
  static constexpr int kMetaOff = kCombOff + kCombBytes;
  static constexpr int kBarOff = kMetaOff + ((kMetaBytes + 15) / 16) * 16;
  static constexpr int kNumBars = 3 * kStages + 2 * kD8AStages + 2 * kD8Windows + kD8MetaSlots;
  static constexpr int kSmemBytes = kBarOff + kNumBars * 8 + 1024 /*align*/;
};

struct D8Params {
  const uint16_t* x;
  const uint16_t* scales;
  const uint32_t* qzeros;
  Epilogue epi;
  uint16_t* y;
  float* partial;
  unsigned* counters;
  unsigned* status;
  const unsigned char* xprep;   // PREP kernels: K / 128 records written by d8_prep_kernel
  int M, K, N;
  int group_size;
  int ntiles;
  int nblk;
  long long units;
  // Row-parallel shard: the epilogue performs the push form of the peer exchange itself (PUSH kernels only).
  unsigned char* const* recv;   // per rank: receive area, 2 parities x world slots x slot_bytes (wire format)
  unsigned* const* pflags;      // per rank: flag array (awq_peer.cuh)
  size_t slot_bytes;
  int rank, world;
};

__device__ __forceinline__ void d8_unpack_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kD8UnpackThreads) : "memory");
}

// Shared-memory matrix descriptor: K-major operand of 8-bit elements, 64-byte rows, 64-byte swizzle, 8-row
// groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_sw64_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(512 >> 4) << 32;                     // stride byte offset: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;                            // descriptor version (sm_100)
  d |= static_cast<uint64_t>(4) << 61;                            // SWIZZLE_64B
  return d;
}

// Instruction descriptor for kind::i8: D int32, A unsigned 8-bit, B signed 8-bit, both K-major.
__host__ __device__ constexpr uint32_t make_i8_idesc(int m, int n) {
  return (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// The four integer MMAs of one unit and half - {hi from tensor memory, raw from shared memory} x two k steps of
// 32 slots - into fresh accumulators, then three commits, under one election.  a_hi: operand columns in tensor
// memory (8 columns per step); a_raw: descriptor of the half's packed bytes as they arrived; b_hi / b_lo:
// descriptors of the activation tiles (a step advances 32 bytes = 2 units of 16 bytes).
__device__ __forceinline__ void tcgen05_mma_i8_unit_commit3_warp(uint32_t d_hi, uint32_t d_raw, uint32_t a_hi, uint64_t a_raw,
                                                                 uint64_t b_hi, uint64_t b_lo, uint32_t idesc,
                                                                 uint32_t idesc_raw, uint32_t bar0, uint32_t bar1,
                                                                 uint32_t bar2) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b32 a, lo, hi;\n\t.reg .b64 d, da;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%0], [%2], %4, %6, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%1], %3, %5, %10, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 a, %2, 8;\n\t  mov.b64 {lo, hi}, %4;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%0], [a], d, %6, p;\n\t"
      "mov.b64 {lo, hi}, %3;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 da, {lo, hi};\n\t"
      "mov.b64 {lo, hi}, %5;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%1], da, d, %10, p;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%8];\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%9];\n\t}"
      ::"r"(d_hi), "r"(d_raw), "r"(a_hi), "l"(a_raw), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(bar0), "r"(bar1), "r"(bar2),
        "r"(idesc_raw)
      : "memory");
}

// The same four MMAs without commits (the first half of a unit).
__device__ __forceinline__ void tcgen05_mma_i8_half_warp(uint32_t d_hi, uint32_t d_raw, uint32_t a_hi, uint64_t a_raw,
                                                         uint64_t b_hi, uint64_t b_lo, uint32_t idesc,
                                                         uint32_t idesc_raw) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b32 a, lo, hi;\n\t.reg .b64 d, da;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%0], [%2], %4, %6, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%1], %3, %5, %7, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 a, %2, 8;\n\t  mov.b64 {lo, hi}, %4;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%0], [a], d, %6, p;\n\t"
      "mov.b64 {lo, hi}, %3;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 da, {lo, hi};\n\t"
      "mov.b64 {lo, hi}, %5;\n\t  add.u32 lo, lo, 2;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::i8 [%1], da, d, %7, p;\n\t}"
      ::"r"(d_hi), "r"(d_raw), "r"(a_hi), "l"(a_raw), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(idesc_raw)
      : "memory");
}

template <int N>
__device__ __forceinline__ void d8_tmem_ld(uint32_t taddr, uint32_t (&v)[N]) {
  static_assert(N == 2 || N == 4 || N == 8 || N == 16, "columns per load");
  if constexpr (N == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
  } else if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr) : "memory");
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
  }
}

// Push form of the row-parallel exchange, per payload word (two adjacent fp16 results of this rank's shard; word w
// of a slot sits at byte 8 w).  d8_push_word stores {payload, epoch} into this rank's slot on every peer;
// d8_collect_word gathers the peers' words for the same position out of this rank's own receive area, adds all
// ranks' values in rank order in fp32 (the arithmetic of peer_allreduce_push_kernel: identical bits on every rank)
// and returns the rounded pair.  Waits are bounded by one limit per call (t_call); on expiry *fail is raised and
// the result is meaningless.  A thread pushes all its words before it collects the first.
constexpr int kD8PushMaxWorld = 8;
__device__ __forceinline__ void d8_push_word(const D8Params& p, unsigned epoch, size_t word, uint32_t payload) {
  const size_t par_off = static_cast<size_t>(epoch & 1u) * p.world;
#pragma unroll
  for (int r = 0; r < kD8PushMaxWorld; ++r)
    if (r < p.world && r != p.rank) st_wire_8(p.recv[r] + (par_off + p.rank) * p.slot_bytes + word * 8, payload, epoch);
}
__device__ __forceinline__ uint32_t d8_collect_word(const D8Params& p, unsigned epoch, unsigned long long t_call,
                                                    unsigned long long limit, volatile int* fail, size_t word,
                                                    uint32_t payload) {
  const size_t par_off = static_cast<size_t>(epoch & 1u) * p.world;
  const unsigned char* slots = p.recv[p.rank] + par_off * p.slot_bytes + word * 8;
  uint2 v[kD8PushMaxWorld];
#pragma unroll
  for (int r = 0; r < kD8PushMaxWorld; ++r) {
    v[r] = make_uint2(payload, epoch);
    if (r < p.world && r != p.rank) v[r] = ld_wire_8(slots + static_cast<size_t>(r) * p.slot_bytes);
  }
  bool ok = true;
#pragma unroll
  for (int r = 0; r < kD8PushMaxWorld; ++r) {
    if (r < p.world && r != p.rank && ok) {
      unsigned spins = 0;
      while (v[r].y != epoch) {
        if ((++spins & 15u) == 0u && (*fail != 0 || clock64() - t_call > limit)) { ok = false; break; }
        v[r] = ld_wire_8(slots + static_cast<size_t>(r) * p.slot_bytes);
      }
    }
  }
  if (!ok) *fail = 1;
  float2 acc = make_float2(0.f, 0.f);
#pragma unroll
  for (int r = 0; r < kD8PushMaxWorld; ++r) {
    if (r < p.world) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[r].x));
      acc.x += f.x;
      acc.y += f.y;
    }
  }
  const __half2 o = __floats2half2_rn(acc.x, acc.y);
  return *reinterpret_cast<const uint32_t*>(&o);
}

// One row's 128 activations of a unit (16 lanes, 8 values each in xv: lane jw holds k = 8 jw .. 8 jw + 7) -> the two
// planes of signed bytes in the order of the weight bytes they multiply, written into the stage's activation tiles,
// and (sx, T) into meta_row[m].  Word j of a column holds k = 8j + e at nibble (e >> 1) + 4 (e & 1), so byte b of that
// word carries k = 8j + {0, 4, 1, 5}[b] in its low nibble and k = 8j + {2, 6, 3, 7}[b] in its high nibble.
template <int MR>
__device__ __forceinline__ void d8_quantise_row(const uint4& xv, int m, int jw, unsigned char* st, int2* meta_row) {
  using Cfg = D8Cfg<MR>;
  float f[8];
  {
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&xv.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&xv.y));
    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&xv.z));
    const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&xv.w));
    f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y; f[4] = f2.x; f[5] = f2.y; f[6] = f3.x; f[7] = f3.y;
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
  for (int off = 1; off < 16; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  // Inf / NaN activations have no integer image: the row's scale becomes 0 * inf = NaN and so does its output.
  const float sx = amax * (1.0f / kD8Range);
  const float inv = amax > 0.f ? static_cast<float>(kD8Range) / amax : 0.f;
  int tq[8], tsum = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int v = __float2int_rn(f[e] * inv);
    v = max(-kD8Range, min(kD8Range, v));
    tq[e] = v;
    tsum += v;
  }
#pragma unroll
  for (int off = 1; off < 16; off <<= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, off);
  // planes: t = 128 * p1 + p2
  uint32_t hi1 = 0u, hi2 = 0u, lo1 = 0u, lo2 = 0u;
  constexpr int kLoK[4] = {0, 4, 1, 5}, kHiK[4] = {2, 6, 3, 7};
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int th = tq[kHiK[b]], tl = tq[kLoK[b]];
    const int h1 = (th + 64) >> 7, l1 = (tl + 64) >> 7;
    hi1 |= static_cast<uint32_t>(h1 & 0xff) << (8 * b);
    hi2 |= static_cast<uint32_t>((th - (h1 << 7)) & 0xff) << (8 * b);
    lo1 |= static_cast<uint32_t>(l1 & 0xff) << (8 * b);
    lo2 |= static_cast<uint32_t>((tl - (l1 << 7)) & 0xff) << (8 * b);
  }
  if (m < MR) {
    // tile row r: 64 bytes, 16-byte chunk c at chunk position c ^ ((r >> 1) & 3)
    const int r1 = Cfg::plane1_row(m), r2 = Cfg::plane2_row(m);
    const uint32_t o1 = static_cast<uint32_t>(r1 * 64 + (((jw >> 2) ^ ((r1 >> 1) & 3)) << 4) + (jw & 3) * 4);
    const uint32_t o2 = static_cast<uint32_t>(r2 * 64 + (((jw >> 2) ^ ((r2 >> 1) & 3)) << 4) + (jw & 3) * 4);
    *reinterpret_cast<uint32_t*>(st + kD8XhiOff + o1) = hi1;
    *reinterpret_cast<uint32_t*>(st + kD8XhiOff + o2) = hi2;
    *reinterpret_cast<uint32_t*>(st + Cfg::kXloOff + o1) = lo1;
    *reinterpret_cast<uint32_t*>(st + Cfg::kXloOff + o2) = lo2;
    if (jw == 0) meta_row[m] = make_int2(__float_as_int(sx), tsum);
  }
}

// The activation planes of a call, once for all CTAs: block b writes the record of k block b (the layout the helper
// warps produce inside a stage: tile Xhi, tile Xlo, then MR x (sx bits, T)).  Used from 5 rows, where the helper
// warps of every CTA repeating this work for each of its units is what bounds the kernel.
template <int MR>
__global__ void __launch_bounds__(128) d8_prep_kernel(const uint16_t* __restrict__ x, unsigned char* __restrict__ out, int M,
                                                      int K) {
  using Cfg = D8Cfg<MR>;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");          // the activations belong to the previous kernel until here
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jw = lane & 15, rsel = lane >> 4;
  const int kb = blockIdx.x;
  unsigned char* rec = out + static_cast<size_t>(kb) * Cfg::kPrepRecBytes;
  for (int r = warp; r < (MR + 1) / 2; r += 4) {
    const int m = 2 * r + rsel;
    uint4 xv = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) xv = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * K + kb * kBlockK + jw * 8));
    d8_quantise_row<MR>(xv, m, jw, rec - kD8XhiOff, reinterpret_cast<int2*>(rec + 2 * Cfg::kXTileBytes));
  }
}

// PREP: the activation planes and (sx, T) of every k block were written by d8_prep_kernel (record layout below);
// the copy producer fetches them with the weights and the helper warps have nothing to do.
template <int MR, bool PUSH, bool PREP>
__global__ void __launch_bounds__(PREP ? kD8Threads - kD8HelperWarps * 32 : kD8Threads, kD8CtasPerSm)
decode_i8_kernel(const __grid_constant__ CUtensorMap map_w, const D8Params p) {
  using Cfg = D8Cfg<MR>;
  constexpr int NT = Cfg::kStages, NA = kD8AStages, NW = kD8Windows, NS = kD8MetaSlots;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ int s_push_fail;
  __shared__ uint32_t s_tmem_base;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  auto stage_addr = [&](int t) { return base + t * Cfg::kStageBytes; };
  float* comb = reinterpret_cast<float*>(base_ptr + Cfg::kCombOff);          // [MR][256]: group 1's sums
  int2* meta = reinterpret_cast<int2*>(base_ptr + Cfg::kMetaOff);            // [NS][MR]: (bits of sx, T)
  const uint32_t bar_base = base + Cfg::kBarOff;
  auto bar_full_tma = [&](int t) { return bar_base + 8u * t; };             // weights, scales, zeros landed
  auto bar_empty = [&](int t) { return bar_base + 8u * (NT + t); };         // 4 unpack warps + the MMA commit
  auto bar_xq_full = [&](int t) { return bar_base + 8u * (2 * NT + t); };   // activation tiles written
  auto bar_a_full = [&](int a) { return bar_base + 8u * (3 * NT + a); };
  auto bar_a_empty = [&](int a) { return bar_base + 8u * (3 * NT + NA + a); };
  auto bar_win_full = [&](int w) { return bar_base + 8u * (3 * NT + 2 * NA + w); };
  auto bar_win_empty = [&](int w) { return bar_base + 8u * (3 * NT + 2 * NA + NW + w); };
  auto bar_meta_full = [&](int s) { return bar_base + 8u * (3 * NT + 2 * NA + 2 * NW + s); };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    s_abort = 0;
    s_push_fail = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_full_tma(t), 1);
      mbar_init(bar_empty(t), kD8UnpackWarps / kD8Groups + 1);
      mbar_init(bar_xq_full(t), 1);
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(bar_a_full(a), kD8UnpackWarps / kD8Groups);
      mbar_init(bar_a_empty(a), 1);
    }
    for (int w = 0; w < NW; ++w) {
      mbar_init(bar_win_full(w), 1);
      mbar_init(bar_win_empty(w), kD8UnpackWarps / kD8Groups);
    }
    for (int s = 0; s < NS; ++s) mbar_init(bar_meta_full(s), 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(static_cast<uint32_t>(kD8TmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  const long long U = p.units, G = gridDim.x;
  const long long u0 = stream_first_unit(blockIdx.x, U, G), u1 = stream_first_unit(blockIdx.x + 1, U, G);
  const int my_units = static_cast<int>(u1 - u0);
  const int nblk = p.nblk;
  constexpr uint32_t kIdesc = make_i8_idesc(128, Cfg::kHiN), kIdescRaw = make_i8_idesc(128, 16);
  const bool sz_by_copy = (p.N & 31) == 0;

  if (warp == 0) {
    // ------------------------------ copy producer ------------------------------
    // Weights, scales and zero words are constant data: the first ring fill starts before the wait on the
    // previous kernel of the stream.  Lanes 2, 3, 4 each issue one of a unit's three copies.
    if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    int tile = static_cast<int>(u0 / nblk);
    int kb = static_cast<int>(u0 - static_cast<long long>(tile) * nblk);
    const int group_blocks = p.group_size / kBlockK;
    auto issue = [&](int gs) {
      const int n0 = tile * kD8BN;
      const int ncols = min(kD8BN, p.N - n0);
      const int t = gs % NT;
      const uint32_t bar = bar_full_tma(t);
      const uint32_t dst = stage_addr(t);
      if (lane == 0) mbar_expect_tx(bar, kD8RawBytes + (sz_by_copy ? ncols * 2 + ncols / 2 : 0));
      if (lane == 2) tma_load_3d(dst + kD8RawOff, &map_w, 0, n0, kb, bar);
      if (sz_by_copy && (lane == 3 || lane == 4)) {
        const int grp = group_blocks == 1 ? kb : kb / group_blocks;
        if (lane == 3) bulk_load(dst + Cfg::kSzOff, p.scales + static_cast<size_t>(grp) * p.N + n0, ncols * 2, bar);
        else bulk_load(dst + Cfg::kSzOff + 512, p.qzeros + static_cast<size_t>(grp) * (p.N >> 3) + (n0 >> 3), ncols / 2, bar);
      }
      if (++kb == nblk) { kb = 0; ++tile; }
    };
    // PREP: the unit's activation tiles (one copy: Xhi and Xlo are adjacent in the record and in the stage) and
    // its (sx, T) rows into ring slot gs % 8 (free for the reason given at the helpers).
    int kbx = static_cast<int>(u0 % nblk);
    auto issue_x = [&](int gs) {
      const int t = gs % NT, s = gs % NS;
      const unsigned char* rec = p.xprep + static_cast<size_t>(kbx) * Cfg::kPrepRecBytes;
      if (lane == 5) {
        mbar_expect_tx(bar_xq_full(t), 2 * Cfg::kXTileBytes);
        bulk_load(stage_addr(t) + kD8XhiOff, rec, 2 * Cfg::kXTileBytes, bar_xq_full(t));
      }
      if (lane == 6) {
        mbar_expect_tx(bar_meta_full(s), Cfg::kPrepMetaBytes);
        bulk_load(base + Cfg::kMetaOff + s * Cfg::kPrepMetaBytes, rec + 2 * Cfg::kXTileBytes, Cfg::kPrepMetaBytes, bar_meta_full(s));
      }
      if (++kbx == nblk) kbx = 0;
    };
    int next = 0;
    for (; next < NT && next < my_units; ++next) issue(next);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if constexpr (PREP) {
      asm volatile("griddepcontrol.wait;" ::: "memory");      // the records are written by the kernel before this one
      for (int gs = 0; gs < next; ++gs) issue_x(gs);
    }
    for (; next < my_units; ++next) {
      if (!mbar_wait(bar_empty(next % NT), static_cast<uint32_t>(next / NT - 1) & 1u, abort_flag, 1)) break;
      issue(next);
      if constexpr (PREP) issue_x(next);
    }
    // Do not leave while a copy may still be writing shared memory: wait (bounded) for the last ring's worth.
    for (int gs = max(0, next - NT); gs < next; ++gs) {
      mbar_wait_timed(bar_full_tma(gs % NT), static_cast<uint32_t>(gs / NT) & 1u);
      if constexpr (PREP) {
        mbar_wait_timed(bar_xq_full(gs % NT), static_cast<uint32_t>(gs / NT) & 1u);
        mbar_wait_timed(bar_meta_full(gs % NS), static_cast<uint32_t>(gs / NS) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    // Warp-uniform loop, one elected lane issues.  Every unit gets fresh accumulators in window gs % 2, which
    // its group has read back (for unit gs - 2) before it signalled this unit's operands.
    for (int gs = 0; gs < my_units; ++gs) {
      const int t = gs % NT, a = gs % NA, w = gs % NW;
      if (!mbar_wait(bar_win_empty(w), (static_cast<uint32_t>(gs / NW) & 1u) ^ 1u, abort_flag, 2)) break;
      if (!mbar_wait(bar_xq_full(t), static_cast<uint32_t>(gs / NT) & 1u, abort_flag, 3)) break;
      if (!mbar_wait(bar_a_full(a), static_cast<uint32_t>(gs / NA) & 1u, abort_flag, 4)) break;
      if (!mbar_wait(bar_full_tma(t), static_cast<uint32_t>(gs / NT) & 1u, abort_flag, 10)) break;   // the raw bytes are an operand
      tcgen05_fence_after();
      const uint32_t win = tmem_base + static_cast<uint32_t>(w * Cfg::kWinCols);
      const uint32_t opd = tmem_base + static_cast<uint32_t>(Cfg::kABase + a * Cfg::kASlot);
      const uint64_t b_hi = make_sw64_desc(stage_addr(t) + kD8XhiOff), b_lo = make_sw64_desc(stage_addr(t) + Cfg::kXloOff);
      const uint64_t a_raw0 = make_sw64_desc(stage_addr(t) + kD8RawOff), a_raw1 = make_sw64_desc(stage_addr(t) + kD8RawOff + 128 * 64);
      tcgen05_mma_i8_half_warp(win, win + Cfg::kHiN, opd, a_raw0, b_hi, b_lo, kIdesc, kIdescRaw);
      tcgen05_mma_i8_unit_commit3_warp(win + Cfg::kHalfCols, win + Cfg::kHalfCols + Cfg::kHiN, opd + Cfg::kASlot / 2, a_raw1,
                                       b_hi, b_lo, kIdesc, kIdescRaw, bar_empty(t), bar_a_empty(a), bar_win_full(w));
    }
    __syncwarp();
  } else if (warp >= kD8HelperWarp0) {
   if constexpr (!PREP) {
    // ------------------------------ activation helpers -------------------------
    // Unit by unit (alternate units per warp): the M rows of this unit's 128 activations -> two planes of
    // signed bytes in the order of the weight bytes they multiply.  Word j of a column holds k = 8j + e at
    // nibble (e >> 1) + 4 (e & 1), so byte b of that word carries k = 8j + {0, 4, 1, 5}[b] in its low nibble and
    // k = 8j + {2, 6, 3, 7}[b] in its high nibble.  Lane = (row parity, word j): 16 lanes share a row.
    asm volatile("griddepcontrol.wait;" ::: "memory");        // the activations belong to the previous kernel until here
    const int jw = lane & 15, rsel = lane >> 4;
    constexpr int RP = (MR + 1) / 2;                          // row pairs
    auto load_x = [&](int gs, uint4 (&xv)[RP]) {
      const long long u = u0 + gs;
      const int tile = static_cast<int>(u / nblk);
      const int kb = static_cast<int>(u - static_cast<long long>(tile) * nblk);
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        const int m = 2 * r + rsel;
        xv[r] = make_uint4(0u, 0u, 0u, 0u);
        if (m < p.M && gs < my_units)
          xv[r] = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.K + kb * kBlockK + jw * 8));
      }
    };
    uint4 xnext[RP];
    const int first = warp - kD8HelperWarp0;
    load_x(first, xnext);
    for (int gs = first; gs < my_units; gs += kD8HelperWarps) {
      const int t = gs % NT, s = gs % NS;
      uint4 xv[RP];
#pragma unroll
      for (int r = 0; r < RP; ++r) xv[r] = xnext[r];
      load_x(gs + kD8HelperWarps, xnext);                     // the next unit's rows travel while this one is processed
      if (gs >= NT && !mbar_wait(bar_empty(t), static_cast<uint32_t>(gs / NT - 1) & 1u, abort_flag, 8)) break;
      // The (sx, T) ring: slot gs % 8 was last used by unit gs - 8, whose fold preceded MMA(gs - 6) (same
      // accumulator window), which preceded the release of stage gs - 5 that this warp has just waited for.
      unsigned char* st = base_ptr + t * Cfg::kStageBytes;
#pragma unroll
      for (int r = 0; r < RP; ++r) d8_quantise_row<MR>(xv[r], 2 * r + rsel, jw, st, meta + s * Cfg::kMetaStride);
      fence_proxy_async();            // the tiles are read by the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_meta_full(s));
        mbar_arrive(bar_xq_full(t));
      }
    }
    __syncwarp();
   }
  } else {
    // ---------------------- mask into tensor memory, then fold accumulators ---------------
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y and the workspace belong to the previous kernel until here
    // PUSH: the call's epoch (advanced by the last CTA of the previous exchange, which has completed by now)
    unsigned push_epoch = 0u;
    unsigned long long push_limit = 0ull, push_t0 = 0ull;
    volatile int* push_fail = &s_push_fail;
    if constexpr (PUSH) {
      const unsigned* my_flags = p.pflags[p.rank];
      push_epoch = my_flags[kArPushEpochOff] + 1u;
      push_limit = wait_limit_cycles(my_flags);
      push_t0 = clock64();
    }
    // This rank's rounded pair (col even) of row m, bias included: what the unfused kernel would have stored.
    auto pair_bits = [&](int col, float a, float b) -> uint32_t {
      __half2 h = __floats2half2_rn(a, b);
      if (p.epi.bias != nullptr) h = __hadd2(h, *reinterpret_cast<const __half2*>(p.epi.bias + col));
      return *reinterpret_cast<const uint32_t*>(&h);
    };
    const int id = tid - 64;                  // 0..255
    const int dq_warp = id >> 5;              // 0..7
    const int lane_q = warp & 3;              // TMEM lane quarter this warp may touch
    const int grp = dq_warp >> 2;             // 0..1; four consecutive warps cover the four quarters
    const int cl0 = lane_q * 32 + lane;       // column within a 128-column half
    const uint32_t lane_addr = static_cast<uint32_t>(lane_q * 32) << 16;
    const int zcols = p.N >> 3;
    bool ok = true;
    int gs = 0;
    while (gs < my_units) {
      const long long u = u0 + gs;
      const int tile = static_cast<int>(u / nblk);
      const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * nblk);
      const int seg_units = min(nblk - kb0, my_units - gs);
      const int n0 = tile * kD8BN;
      int ncol[2];
      bool nval[2];
      uint32_t zsh[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ncol[h] = n0 + h * 128 + cl0;
        nval[h] = ncol[h] < p.N;
        zsh[h] = awq_slot_shift(static_cast<uint32_t>(ncol[h] & 7));
      }
      uint32_t sc[2] = {0u, 0u}, zw[2] = {0u, 0u};
      int sz_group = -1;
      float acc[2][MR];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int m = 0; m < MR; ++m) acc[h][m] = 0.f;
      int pend = -1;
      float pend_s[2] = {0.f, 0.f};
      int pend_z[2] = {0, 0};

      // acc[h][m] += s * sx[m] * ((128 Dhi[m] + Dhi[MR + m]) / 16 + 128 Dlo[m] + Dlo[MR + m] - z T[m])
      auto fold_pending = [&]() {
        if (pend < 0) return;
        const int w = pend % NW, s = pend % NS;
        if (ok && !mbar_wait(bar_meta_full(s), static_cast<uint32_t>(pend / NS) & 1u, abort_flag, 9)) ok = false;
        if (ok && !mbar_wait(bar_win_full(w), static_cast<uint32_t>(pend / NW) & 1u, abort_flag, 6)) ok = false;
        if constexpr (MR == 8) {
          // Four rows at a time: the two planes of rows 4 c .. 4 c + 3 are eight adjacent accumulator columns.
          if (ok) {
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t vh[2][8], vx[2][8], vr[2][8];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t win = tmem_base + lane_addr + static_cast<uint32_t>(w * Cfg::kWinCols + h * Cfg::kHalfCols);
                d8_tmem_ld<8>(win + 8 * c, vh[h]);                  // hi x (activations of the high nibbles)
                d8_tmem_ld<8>(win + 16 + 8 * c, vx[h]);             // hi x (activations of the low nibbles)
                d8_tmem_ld<8>(win + Cfg::kHiN + 8 * c, vr[h]);      // raw x (activations of the low nibbles)
              }
              tcgen05_wait_ld();
              if (c == 1) {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_win_empty(w));
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int m = 4 * c + q;
                const int2 mt = meta[s * Cfg::kMetaStride + m];                  // same address in every lane: a broadcast
                const float sx = __int_as_float(mt.x);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int dhi = (static_cast<int>(vh[h][2 * q]) << 7) + static_cast<int>(vh[h][2 * q + 1]);
                  const int dlo = ((static_cast<int>(vr[h][2 * q]) - static_cast<int>(vx[h][2 * q])) << 7) +
                                  (static_cast<int>(vr[h][2 * q + 1]) - static_cast<int>(vx[h][2 * q + 1]));
                  const int val = (dhi >> 4) + dlo - pend_z[h] * mt.y;
                  acc[h][m] = fmaf(pend_s[h] * sx, static_cast<float>(val), acc[h][m]);
                }
              }
            }
          }
        } else if (ok) {
          tcgen05_fence_after();
          uint32_t vh[2][2 * MR], vx[2][2 * MR], vr[2][2 * MR];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t win = tmem_base + lane_addr + static_cast<uint32_t>(w * Cfg::kWinCols + h * Cfg::kHalfCols);
            d8_tmem_ld<2 * MR>(win, vh[h]);             // hi x (activations of the high nibbles)
            d8_tmem_ld<2 * MR>(win + 8, vx[h]);         // hi x (activations of the low nibbles): rows 8.. of the B tile
            d8_tmem_ld<2 * MR>(win + 16, vr[h]);        // raw x (activations of the low nibbles)
          }
          tcgen05_wait_ld();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_win_empty(w));
#pragma unroll
          for (int m = 0; m < MR; ++m) {
            const int2 mt = meta[s * Cfg::kMetaStride + m];                  // same address in every lane: a broadcast
            const float sx = __int_as_float(mt.x);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int dhi = (static_cast<int>(vh[h][m]) << 7) + static_cast<int>(vh[h][MR + m]);    // a multiple of 16
              // raw = hi + lo byte by byte, so (raw - hi) . x = lo . x, plane by plane
              const int dlo = ((static_cast<int>(vr[h][m]) - static_cast<int>(vx[h][m])) << 7) +
                              (static_cast<int>(vr[h][MR + m]) - static_cast<int>(vx[h][MR + m]));
              const int val = (dhi >> 4) + dlo - pend_z[h] * mt.y;
              acc[h][m] = fmaf(pend_s[h] * sx, static_cast<float>(val), acc[h][m]);
            }
          }
        }
        pend = -1;
      };

      for (int j = 0; j < seg_units; ++j, ++gs) {
        if ((gs & (kD8Groups - 1)) != grp) continue;             // another group's unit
        const int t = gs % NT, a = gs % NA;
        const uint32_t ph = static_cast<uint32_t>(gs / NT) & 1u, pha = static_cast<uint32_t>(gs / NA) & 1u;
        fold_pending();                                          // this group's previous unit, two units back
        if (!sz_by_copy) {
          const int qgrp = ((kb0 + j) * kBlockK) / p.group_size;
          if (qgrp != sz_group) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              sc[h] = nval[h] ? __ldg(p.scales + static_cast<size_t>(qgrp) * p.N + ncol[h]) : 0u;
              zw[h] = nval[h] ? __ldg(p.qzeros + static_cast<size_t>(qgrp) * zcols + (ncol[h] >> 3)) : 0u;
            }
            sz_group = qgrp;
          }
        }
        if (ok && !mbar_wait(bar_full_tma(t), ph, abort_flag, 5)) ok = false;
        if (!ok) continue;
        const unsigned char* stage = base_ptr + t * Cfg::kStageBytes;
        if (sz_by_copy) {
          // Columns beyond N read stale shared memory here; their lanes of the product are never stored.
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            sc[h] = reinterpret_cast<const uint16_t*>(stage + Cfg::kSzOff)[h * 128 + cl0];
            zw[h] = reinterpret_cast<const uint32_t*>(stage + Cfg::kSzOff + 512)[(h * 128 + cl0) >> 3];
          }
        }
        if (!mbar_wait(bar_a_empty(a), pha ^ 1u, abort_flag, 7)) {
          ok = false;
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty(t));
          continue;
        }
        tcgen05_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int cl = h * 128 + cl0;
          uint4 r[4];
          const uint32_t swz = static_cast<uint32_t>((cl >> 1) & 3);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            r[c] = *reinterpret_cast<const uint4*>(stage + kD8RawOff + cl * 64 + ((static_cast<uint32_t>(c) ^ swz) << 4));
          if (h == 1) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(t));            // the stage's packed weights are in registers
          }
          const uint32_t a_addr = tmem_base + lane_addr + static_cast<uint32_t>(Cfg::kABase + a * Cfg::kASlot + h * (Cfg::kASlot / 2));
          uint32_t o[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            o[4 * c + 0] = r[c].x & 0xf0f0f0f0u; o[4 * c + 1] = r[c].y & 0xf0f0f0f0u;
            o[4 * c + 2] = r[c].z & 0xf0f0f0f0u; o[4 * c + 3] = r[c].w & 0xf0f0f0f0u;
          }
          tcgen05_st_32x32b_x16(a_addr, o);
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_a_full(a));
        pend = gs;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          pend_s[h] = __half2float(__ushort_as_half(static_cast<unsigned short>(sc[h])));
          pend_z[h] = static_cast<int>((zw[h] >> zsh[h]) & 0xFu);
        }
      }
      fold_pending();

      // ------------------------------ segment epilogue ------------------------
      d8_unpack_warps_sync();
      if (grp != 0) {
        float* cb = comb;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int m = 0; m < MR; ++m) cb[m * kD8BN + h * 128 + cl0] = acc[h][m];
      }
      d8_unpack_warps_sync();
      const long long tile_u0 = static_cast<long long>(tile) * nblk;
      const int c_first = stream_cta_of(tile_u0, U, G);
      const int c_last = stream_cta_of(tile_u0 + nblk - 1, U, G);
      const int nc = c_last - c_first + 1;
      const int slot = static_cast<int>(blockIdx.x) - c_first;
      const bool direct = (nc == 1);
      if (grp == 0) {
        if (PUSH && direct) {
          // Exchange in the epilogue: an even lane owns the pair (its column, its neighbour's); all of a thread's
          // words leave for the peers before it collects the first of theirs.
          uint32_t pay[2][MR];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int m = 0; m < MR; ++m) {
              pay[h][m] = 0u;
              if (m < p.M) {                               // warp-uniform
                const float val = acc[h][m] + comb[m * kD8BN + h * 128 + cl0];
                const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                if (nval[h] && (lane & 1) == 0) {
                  pay[h][m] = pair_bits(ncol[h], val, other);
                  d8_push_word(p, push_epoch, (static_cast<size_t>(m) * p.N + ncol[h]) >> 1, pay[h][m]);
                }
              }
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int m = 0; m < MR; ++m) {
              if (m < p.M && nval[h] && (lane & 1) == 0) {
                const size_t at = static_cast<size_t>(m) * p.N + ncol[h];
                *reinterpret_cast<uint32_t*>(p.y + at) =
                    d8_collect_word(p, push_epoch, push_t0, push_limit, push_fail, at >> 1, pay[h][m]);
              }
            }
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int m = 0; m < MR; ++m) {
              if (m < p.M) {                                 // warp-uniform
                const float val = acc[h][m] + comb[m * kD8BN + h * 128 + cl0];
                if (direct) epilogue_store_lane(p.y, p.epi, m, p.N, ncol[h], val, nval[h]);
                else if (nval[h]) __stcg(p.partial + (static_cast<size_t>(slot) * p.M + m) * p.N + ncol[h], val);
              }
            }
          }
        }
      }
      if (!direct) {
        __threadfence();
        d8_unpack_warps_sync();
        if (id == 0) {
          const unsigned prev = atomicAdd(&p.counters[tile], 1u);
          const int last = (prev == static_cast<unsigned>(nc - 1));
          if (last) p.counters[tile] = 0u;   // every contributor has arrived: leave the counter clean
          s_last = last;
        }
        d8_unpack_warps_sync();
        if (s_last) {
          __threadfence();
          const int ncols = min(kD8BN, p.N - n0);
          const int pairs = ncols >> 1;
          const size_t slot_stride = static_cast<size_t>(p.M) * p.N;
          for (int i = id; i < p.M * pairs; i += kD8UnpackThreads) {
            const int row = i / pairs;
            const int col = n0 + 2 * (i - row * pairs);
            const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
            // (the plain loop: loading the slots in batches, as the other kernels' reductions do, measured 0.3-0.5 us
            // slower here on tiles shared by two CTAs, which is what the unsharded model shapes have)
            float2 sum = __ldcg(reinterpret_cast<const float2*>(src));
            for (int s = 1; s < nc; ++s) {
              const float2 v = __ldcg(reinterpret_cast<const float2*>(src + s * slot_stride));
              sum.x += v.x;
              sum.y += v.y;
            }
            if constexpr (PUSH) {
              const uint32_t mine = pair_bits(col, sum.x, sum.y);
              const size_t at = static_cast<size_t>(row) * p.N + col;
              d8_push_word(p, push_epoch, at >> 1, mine);
              *reinterpret_cast<uint32_t*>(p.y + at) =
                  d8_collect_word(p, push_epoch, push_t0, push_limit, push_fail, at >> 1, mine);
            } else {
              epilogue_store_pair(p.y, p.epi, row, p.N, col, sum.x, sum.y);
            }
          }
        }
        d8_unpack_warps_sync();   // s_last is rewritten by the next straddling segment
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(kD8TmemCols))
                 : "memory");
  }
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, 0x400u | static_cast<unsigned>(s_abort));
  if constexpr (PUSH) {
    // The last CTA closes the exchange: the epoch advances once per call (device memory: graphs replay).  Every
    // CTA read the old epoch after the barrier above at the latest, and the last one writes after all have counted.
    if (tid == 0) {
      unsigned* my_flags = p.pflags[p.rank];
      const unsigned epoch = my_flags[kArPushEpochOff] + 1u;
      if (s_push_fail != 0 || s_abort != 0) atomicCAS(my_flags + kArStatusOff, 0u, 3u);
      __threadfence();
      const unsigned prev = atomicAdd(my_flags + kArPushBlocksOff, 1u);
      if (prev == gridDim.x - 1) {
        my_flags[kArPushBlocksOff] = 0u;
        my_flags[kArPushEpochOff] = epoch;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
// Number of CTAs.  Two per SM, except that when a slightly smaller grid is a whole multiple of the column tiles,
// that grid is taken: every tile is then shared by the same number of CTAs and no CTA straddles two tiles (one
// epilogue per CTA instead of two; measured 27.4 -> 25.7 us on 28672 -> 8192, 13.7 -> 10.7 us on 7168 -> 8192).
static long long decode_grid(int sm_count, long long units, int ntiles) {
  const long long ctas = static_cast<long long>(kD8CtasPerSm) * sm_count;
  if (units <= ctas) return units;
  if (ntiles <= ctas) {
    const long long g = (ctas / ntiles) * ntiles;
    if (g * 10 >= ctas * 9) return g;
  }
  return ctas;
}

// Largest number of CTAs that share one column tile (= partial slots needed).
static int decode_slots(int K, int N, int sm_count) {
  const int nblk = K / kBlockK, ntiles = (N + kD8BN - 1) / kD8BN;
  const long long U = static_cast<long long>(ntiles) * nblk;
  const long long G = decode_grid(sm_count, U, ntiles);
  int worst = 1;
  for (int t = 0; t < ntiles; ++t) {
    const long long a = static_cast<long long>(t) * nblk;
    const int nc = stream_cta_of(a + nblk - 1, U, G) - stream_cta_of(a, U, G) + 1;
    if (nc > worst) worst = nc;
  }
  return worst;
}

size_t decode_workspace_bytes(int M, int K, int N, int sm_count) {
  if (M < 1 || K < kBlockK || N < 8) return 0;
  const int slots = decode_slots(K, N, sm_count);
  const size_t prep = static_cast<size_t>(K / kBlockK) * D8Cfg<8>::kPrepRecBytes;   // the planes' records (largest form)
  return kGemvMaxCounters * sizeof(unsigned) + (slots > 1 ? static_cast<size_t>(slots) * M * N * sizeof(float) : 0) + prep;
}

template <int MR, bool PUSH, bool PREP>
static int launch_decode_i8(const void* packed, D8Params p, int grid, EncodeTiledFn encode, cudaStream_t stream,
                            bool overlap_previous, int max_smem_optin) {
  using Cfg = D8Cfg<MR>;
  if (Cfg::kSmemBytes > max_smem_optin) return AWQ_B200_ERR_TOO_LARGE;
  CUtensorMap mw;
  {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.K / kBlockK)};
    const cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(p.N) * 64};
    const cuuint32_t box[3] = {64, kD8BN, 1};
    const CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_64B;
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(packed), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  AWQ_CUDA_TRY(cudaFuncSetAttribute(decode_i8_kernel<MR, PUSH, PREP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  // two CTAs of ~100 KB per SM: ask for the largest shared-memory carve-out
  AWQ_CUDA_TRY(cudaFuncSetAttribute(decode_i8_kernel<MR, PUSH, PREP>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    cudaSharedmemCarveoutMaxShared));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(PREP ? kD8Threads - kD8HelperWarps * 32 : kD8Threads);   // no helper warps behind the planes' kernel
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (overlap_previous) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if constexpr (PREP) {
    // The planes first (it takes the caller's overlap choice); the main kernel may always start early behind it:
    // until its own wait it touches nothing but the weights, which the planes' kernel has waited for as well.
    cudaLaunchConfig_t pc = cfg;
    pc.gridDim = dim3(p.nblk);
    pc.blockDim = dim3(128);
    pc.dynamicSmemBytes = 0;
    AWQ_CUDA_TRY(cudaLaunchKernelEx(&pc, d8_prep_kernel<MR>, p.x, const_cast<unsigned char*>(p.xprep), p.M, p.K));
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_i8_kernel<MR, PUSH, PREP>, mw, p));
  return AWQ_B200_OK;
}

struct D8PushArgs {
  void* const* recv;
  void* const* flags;
  size_t slot_elems;
  int rank, world;
};

static int decode_i8_run(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                         void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                         cudaStream_t stream, unsigned flags, const D8PushArgs* push) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size)) return st;
  if (M < 1 || M > kD8MaxRows) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) || !aligned16(y))
    return AWQ_B200_ERR_ALIGN;
  if (int st = check_epilogue(epi, N)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;
  EncodeTiledFn encode;
  if (int st = get_encode(&encode)) return st;
  const int ntiles = (N + kD8BN - 1) / kD8BN;
  if (ntiles > kGemvMaxCounters - 1) return AWQ_B200_ERR_TOO_LARGE;
  if (!workspace || workspace_bytes < decode_workspace_bytes(M, K, N, di.sm_count)) return AWQ_B200_ERR_WORKSPACE;
  if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
  D8Params p;
  p.x = static_cast<const uint16_t*>(x);
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.epi = epi;
  p.y = static_cast<uint16_t*>(y);
  p.counters = static_cast<unsigned*>(workspace);
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kGemvMaxCounters * sizeof(unsigned));
  p.status = static_cast<unsigned*>(workspace) + (kGemvMaxCounters - 1);
  {
    const int slots = decode_slots(K, N, di.sm_count);
    p.xprep = reinterpret_cast<const unsigned char*>(p.partial) + (slots > 1 ? static_cast<size_t>(slots) * M * N * sizeof(float) : 0);
  }
  p.M = M; p.K = K; p.N = N;
  p.group_size = group_size;
  p.ntiles = ntiles;
  p.nblk = K / kBlockK;
  p.units = static_cast<long long>(ntiles) * p.nblk;
  const int grid = static_cast<int>(decode_grid(di.sm_count, p.units, ntiles));
  const bool overlap = (flags & AWQ_B200_OVERLAP_PREVIOUS) != 0;
  p.recv = nullptr; p.pflags = nullptr; p.slot_bytes = 0; p.rank = 0; p.world = 0;
  if (push != nullptr) {
    if (!push->recv || !push->flags) return AWQ_B200_ERR_NULL;
    if (push->world < 2 || push->world > 8 || push->rank < 0 || push->rank >= push->world) return AWQ_B200_ERR_SHAPE;
    if (static_cast<size_t>(M) * N > push->slot_elems) return AWQ_B200_ERR_TOO_LARGE;
    if (epi.residual != nullptr || epi.gated) return AWQ_B200_ERR_SHAPE;      // the exchanged value is the plain sum
    p.recv = reinterpret_cast<unsigned char* const*>(push->recv);
    p.pflags = reinterpret_cast<unsigned* const*>(push->flags);
    p.slot_bytes = push->slot_elems * 4;
    p.rank = push->rank;
    p.world = push->world;
    if (M <= 1) return launch_decode_i8<1, true, false>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
    if (M <= 2) return launch_decode_i8<2, true, false>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
    if (M <= 4) return launch_decode_i8<4, true, true>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
    return launch_decode_i8<8, true, true>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  }
  if (M <= 1) return launch_decode_i8<1, false, false>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  if (M <= 2) return launch_decode_i8<2, false, false>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  if (M <= 4) return launch_decode_i8<4, false, true>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  return launch_decode_i8<8, false, true>(packed, p, grid, encode, stream, overlap, di.max_smem_optin);
}

int decode_i8_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                       void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream, unsigned flags) {
  return decode_i8_run(x, packed, scales, qzeros, epi, y, M, K, N, group_size, workspace, workspace_bytes, stream, flags,
                       nullptr);
}

}  // namespace awq

extern "C" {

size_t awq_b200_decode_workspace_bytes(int M, int K, int N) {
  awq::DeviceInfo di;
  int sm = 148;
  if (awq::device_info(&di) == AWQ_B200_OK) sm = di.sm_count;
  return awq::decode_workspace_bytes(M, K, N, sm);
}

int awq_b200_decode_i8(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                       void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                       awq_b200_stream_t stream, unsigned flags) {
  return awq::decode_i8_dispatch(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0},
                                 y, M, K, N, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), flags);
}

// awq_b200_decode_i8 for a row-parallel shard, with the push form of the peer exchange (awq_b200_peer_allreduce_push)
// performed by the kernel's epilogue: y receives the SUM over the ranks.
int awq_b200_decode_i8_push(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                            const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                            size_t workspace_bytes, void* const* recv, void* const* flags, size_t slot_elems, int rank,
                            int world, awq_b200_stream_t stream, unsigned call_flags) {
  const awq::D8PushArgs push{recv, flags, slot_elems, rank, world};
  return awq::decode_i8_run(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M,
                            K, N, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), call_flags,
                            &push);
}

}  // extern "C"
