// Decode path for 1 <= M <= 16 rows of a large matrix on tcgen05: the packed nibbles go to tensor memory as
// UNSCALED codes (five logic operations per packed word instead of the thirteen that build the exact fp16
// weight), and scale / zero point are applied in fp32 once per 128-k unit when its accumulator is read back.
//
//   y[m, n] = sum over units u of column tile T(n):   s[u, n] * ( D_u[n, m] - H_u[m] - z[u, n] * S_u[m] )
//   D_u[n, m] = sum_{k in u} code[k, n] * x[m, k]      tcgen05.mma, A = codes from tensor memory (lane = column n),
//                                                      B = the activation rows from shared memory, fp32 in TMEM
//   code[k, n] = c(k) + q[k, n],  c(k) = 1024 for k % 8 in {0, 1, 4, 5}, 64 otherwise  (the nibble or-ed into the
//                                                      mantissa of 2^10 or 2^6: `unpack_codes`)
//   S_u[m] = sum_{k in u} x[m, k],   H_u[m] = sum_{k in u} c(k) * x[m, k]              one warp, fp32, from the
//                                                      activation tile the copy pipeline already brought in
// The weights are multiplied un-rounded (s * (q - z) in fp32), the choice the reference's own GEMV makes
// (LLMQRT/runtime_refact/csrc/awq/gemv.cu:138); measured distance to the fp16-weight oracle ~3e-4 of max|y|.
//
// Work distribution is the split-K stream of the exact-weight kernel (awq_skinny.cu): unit = 256 columns x 128 k
// (16 KiB of packed weights), CTA b owns units [b*U/G, (b+1)*U/G) of the flattened (column tile, k block)
// sequence, one CTA per SM, one copy pipeline that never drains; a column tile that straddles CTAs is finished
// through fp32 partials added in CTA (= k) order by the last contributor.  Deterministic; a row's bits do not
// depend on M (rows are independent columns of the MMA's B operand and the partition depends on (K, N) only).
//
// Warps: 0 / 18 copy producers (even / odd units), 1 / 19 MMA issuers (low / high 128 columns), 20 activation
// sums, 2..17 unpack (two groups of eight that take the units in turn) and read the accumulators back.
// Every unit has its own accumulator window in tensor memory (4 windows x 2 halves x 16 columns), so a group
// reads unit u's window only after it has unpacked unit u + 2: by then the MMAs of u have long finished and
// nobody waits for a tensor-memory round trip.  TMEM columns: [0, 128) windows, [128, 512) three A slots.
// Every mbarrier wait is bounded (see awq_ptx.cuh).
#include "awq_gemv_common.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kDcUnpackWarps = 16;
constexpr int kDcUnpackThreads = kDcUnpackWarps * 32;
constexpr int kDcThreads = 64 + kDcUnpackThreads + 64 + 32;
constexpr int kDcProducer2Warp = 18, kDcIssuer2Warp = 19, kDcSumsWarp = 20;
constexpr int kDcBN = 256;                       // output columns per tile
constexpr int kDcRawBytes = kDcBN * 64;          // one unit of packed weights: [256 columns][64 bytes], 64-byte swizzle
constexpr int kDcMT = 16;                        // MMA N extent = activation rows per box (rows beyond M are zero-filled)
constexpr int kDcXHalfBytes = kDcMT * 128;       // 16 rows x 64 k
constexpr int kDcXBytes = 2 * kDcXHalfBytes;     // 4 KiB, already a multiple of 1024
constexpr int kDcRawOff = kDcXBytes;
constexpr int kDcSzOff = kDcRawOff + kDcRawBytes;   // 256 fp16 scales, then 32 qzeros words
constexpr int kDcStageBytes = kDcSzOff + 1024;
constexpr int kDcStages = 8;
constexpr int kDcWindows = 4;                    // accumulator windows (units in flight between MMA and read-back)
constexpr int kDcABase = kDcWindows * 2 * kDcMT; // 128
constexpr int kDcAStages = 3;
constexpr int kDcSumSlots = 16;                  // ring of per-unit activation sums; must be >= kDcStages + 2
static_assert(kDcABase + kDcAStages * 128 == 512, "tensor memory is used in full");
static_assert(kDcSumSlots >= kDcStages + 2 && kDcStages % 2 == 0, "see the sums ring / two producers");

template <int MR> struct DcCfg {
  static_assert(MR == 1 || MR == 2 || MR == 4 || MR == 8 || MR == 16, "rows read back per unit");
  static constexpr int kCombBytes = 2 * kDcBN * MR * 4;           // group 1's sums of a segment, double-buffered
  static constexpr int kSumsBytes = kDcSumSlots * MR * 8;         // (S, H) per unit and row
  static constexpr int kCombOff = kDcStages * kDcStageBytes;
  static constexpr int kSumsOff = kCombOff + kCombBytes;
  static constexpr int kBarOff = kSumsOff + ((kSumsBytes + 15) / 16) * 16;
  static constexpr int kNumBars = 2 * kDcStages + 2 * kDcAStages + 4 * kDcWindows + kDcSumSlots;
  static constexpr int kSmemBytes = kBarOff + kNumBars * 8 + 1024 /*align*/;
};

struct DcParams {
  const uint16_t* scales;
  const uint32_t* qzeros;
  Epilogue epi;
  uint16_t* y;
  float* partial;        // [slot][M][N] fp32, used by column tiles that straddle CTAs
  unsigned* counters;    // one arrival counter per column tile
  unsigned* status;
  int M, K, N;
  int group_size;
  int ntiles;            // column tiles
  int nblk;              // K / 128
  long long units;       // ntiles * nblk
};

__device__ __forceinline__ void unpack_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kDcUnpackThreads) : "memory");
}

// Eight k-steps of A-from-tensor-memory MMAs into a fresh accumulator, then three commits (activation stage
// free, A slot free, accumulator window complete), issued by one elected lane under a single election.
__device__ __forceinline__ void tcgen05_mma_f16_ts_k8_commit3_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                                   uint32_t step_lo, uint32_t half_lo, uint32_t idesc,
                                                                   uint32_t bar0, uint32_t bar1, uint32_t bar2) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b32 a, lo, hi, lo0;\n\t.reg .b64 d;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"                      // first step overwrites the window
      "elect.sync _|e, 0xffffffff;\n\t"
      "mov.b64 {lo0, hi}, %2;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %5, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 a, %1, 8;\n\t  add.u32 lo, lo0, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo0, %4;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%8];\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(step_lo), "r"(half_lo), "r"(idesc), "r"(bar0), "r"(bar1), "r"(bar2)
      : "memory");
}

// MR consecutive 32-bit columns of this thread's tensor-memory lane.
template <int MR>
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, uint32_t (&v)[MR]) {
  if constexpr (MR == 1) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v[0]) : "r"(taddr) : "memory");
  } else if constexpr (MR == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
  } else if constexpr (MR == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
  } else if constexpr (MR == 8) {
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

template <int MR>
__global__ void __launch_bounds__(kDcThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const DcParams p) {
  using Cfg = DcCfg<MR>;
  constexpr int NT = kDcStages, NA = kDcAStages, NW = kDcWindows, NS = kDcSumSlots;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ uint32_t s_tmem_base;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  auto stage_addr = [&](int t) { return base + t * kDcStageBytes; };
  float* comb = reinterpret_cast<float*>(base_ptr + Cfg::kCombOff);          // [2][MR][256]
  float2* sums = reinterpret_cast<float2*>(base_ptr + Cfg::kSumsOff);        // [NS][MR]
  const uint32_t bar_base = base + Cfg::kBarOff;
  auto bar_full_tma = [&](int t) { return bar_base + 8u * t; };
  auto bar_empty_tma = [&](int t) { return bar_base + 8u * (NT + t); };     // 8 unpack warps + 2 MMA commits + sums warp
  auto bar_a_full = [&](int a) { return bar_base + 8u * (2 * NT + a); };
  auto bar_a_empty = [&](int a) { return bar_base + 8u * (2 * NT + NA + a); };
  auto bar_win_full = [&](int h, int w) { return bar_base + 8u * (2 * NT + 2 * NA + h * NW + w); };
  auto bar_win_empty = [&](int h, int w) { return bar_base + 8u * (2 * NT + 2 * NA + 2 * NW + h * NW + w); };
  auto bar_sums_full = [&](int s) { return bar_base + 8u * (2 * NT + 2 * NA + 4 * NW + s); };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    s_abort = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_full_tma(t), 1);
      mbar_init(bar_empty_tma(t), kDcUnpackWarps / 2 + 2 + 1);
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(bar_a_full(a), kDcUnpackWarps / 2);
      mbar_init(bar_a_empty(a), 2);
    }
    for (int h = 0; h < 2; ++h) {
      for (int w = 0; w < NW; ++w) {
        mbar_init(bar_win_full(h, w), 1);
        mbar_init(bar_win_empty(h, w), 4);
      }
    }
    for (int s = 0; s < NS; ++s) mbar_init(bar_sums_full(s), 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(512u)
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
  constexpr uint32_t kIdesc = make_f16_idesc(128, kDcMT);
  // Bulk copies need 16-byte aligned, 16-byte sized row segments of scales and qzeros: N % 32 == 0.
  const bool sz_by_copy = (p.N & 31) == 0;

  if (warp == 0 || warp == kDcProducer2Warp) {
    // ------------------------------ copy producers ----------------------------
    // Warp-uniform loops; lanes 0..4 each issue one of a unit's five copies.  The weight-side copies of the
    // first ring fill are constant data and start before the wait on the previous kernel of the stream; the
    // activation boxes follow it.
    const int my_parity = warp == 0 ? 0 : 1;
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    int tile, kb;
    {
      const long long u = u0 + my_parity;
      tile = static_cast<int>(u / nblk);
      kb = static_cast<int>(u - static_cast<long long>(tile) * nblk);
    }
    const int group_blocks = p.group_size / kBlockK;
    auto advance = [&]() {
      kb += 2;
      while (kb >= nblk) { kb -= nblk; ++tile; }
    };
    auto issue = [&](int gs, int tile_, int kb_, bool weights, bool activations) {
      const int n0 = tile_ * kDcBN;
      const int ncols = min(kDcBN, p.N - n0);
      const int t = gs % NT;
      const uint32_t bar = bar_full_tma(t);
      const uint32_t dst = stage_addr(t);
      if (weights) {
        if (lane == 0)
          mbar_expect_tx(bar, kDcXBytes + kDcRawBytes + (sz_by_copy ? ncols * 2 + ncols / 2 : 0));
        if (lane == 2) tma_load_3d(dst + kDcRawOff, &map_w, 0, n0, kb_, bar);
        if (sz_by_copy && (lane == 3 || lane == 4)) {
          const int grp = group_blocks == 1 ? kb_ : kb_ / group_blocks;
          if (lane == 3) bulk_load(dst + kDcSzOff, p.scales + static_cast<size_t>(grp) * p.N + n0, ncols * 2, bar);
          else bulk_load(dst + kDcSzOff + 512, p.qzeros + static_cast<size_t>(grp) * (p.N >> 3) + (n0 >> 3), ncols / 2, bar);
        }
      }
      if (activations && lane < 2) tma_load_2d(dst + lane * kDcXHalfBytes, &map_x, kb_ * kBlockK + lane * 64, 0, bar);
    };
    const int tile_first = tile, kb_first = kb;
    for (int gs = my_parity; gs < NT && gs < my_units; gs += 2) { issue(gs, tile, kb, true, false); advance(); }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
      const int tile_next = tile, kb_next = kb;
      tile = tile_first; kb = kb_first;
      for (int gs = my_parity; gs < NT && gs < my_units; gs += 2) { issue(gs, tile, kb, false, true); advance(); }
      tile = tile_next; kb = kb_next;
    }
    int next = NT + my_parity;
    for (; next < my_units; next += 2) {
      if (!mbar_wait(bar_empty_tma(next % NT), static_cast<uint32_t>(next / NT - 1) & 1u, abort_flag, 1)) break;
      issue(next, tile, kb, true, true);
      advance();
    }
    // Do not leave while a copy of this warp may still be writing shared memory: wait (bounded) for the last
    // ring's worth of its units to land.
    const int issued_end = next < my_units ? next : my_units;
    for (int gs = my_parity; gs < issued_end; gs += 2)
      if (gs + NT >= issued_end) mbar_wait_timed(bar_full_tma(gs % NT), static_cast<uint32_t>(gs / NT) & 1u);
    __syncwarp();
  } else if (warp == 1 || warp == kDcIssuer2Warp) {
    // ------------------------------ MMA issuers --------------------------------
    // One warp per 128-column half; warp-uniform loop, one elected lane issues.  Every unit gets a fresh
    // accumulator window; the window is reused four units later, once its read-back has been signalled.
    const int h = warp == 1 ? 0 : 1;
    for (int gs = 0; gs < my_units; ++gs) {
      const int t = gs % NT, a = gs % NA, w = gs % NW;
      if (!mbar_wait(bar_win_empty(h, w), (static_cast<uint32_t>(gs / NW) & 1u) ^ 1u, abort_flag, 2)) break;
      if (!mbar_wait(bar_full_tma(t), static_cast<uint32_t>(gs / NT) & 1u, abort_flag, 3)) break;
      if (!mbar_wait(bar_a_full(a), static_cast<uint32_t>(gs / NA) & 1u, abort_flag, 4)) break;
      tcgen05_fence_after();
      tcgen05_mma_f16_ts_k8_commit3_warp(tmem_base + static_cast<uint32_t>((w * 2 + h) * kDcMT),
                                         tmem_base + static_cast<uint32_t>(kDcABase + a * 128 + h * 64),
                                         make_sw128_desc(stage_addr(t)), 32u >> 4, kDcXHalfBytes >> 4, kIdesc,
                                         bar_empty_tma(t), bar_a_empty(a), bar_win_full(h, w));
    }
    __syncwarp();
  } else if (warp == kDcSumsWarp) {
    // ------------------------------ activation sums ----------------------------
    // Per unit and row: S = sum of the 128 activations, H = sum of c(k) * x[k].  A row is two 128-byte lines
    // of the (swizzled) activation tile; the swizzle permutes whole 16-byte chunks of 8 consecutive k, so any
    // chunk contributes elements 0, 1, 4, 5 to the 1024-sum and 2, 3, 6, 7 to the 64-sum wherever it lies.
    // Lane = (row, part): P lanes share a row's 16 chunks and add up through shuffles.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int P = (32 / MR) < 16 ? (32 / MR) : 16;    // lanes per row
    constexpr int CPL = 16 / P;                           // chunks per lane
    const int row = lane / P, part = lane % P;
    const bool active = row < MR;
    for (int gs = 0; gs < my_units; ++gs) {
      const int t = gs % NT, s = gs % NS;
      if (!mbar_wait(bar_full_tma(t), static_cast<uint32_t>(gs / NT) & 1u, abort_flag, 8)) break;
      const unsigned char* xt = base_ptr + t * kDcStageBytes;
      // The 16 chunk sums of a row are added as a balanced binary tree over the chunk index whatever MR is
      // (inside a lane over its aligned block of chunks, then across lanes by butterfly), so a row's sums -
      // and with them its output bits - do not depend on how many rows the call has.
      float lo_c[CPL], hi_c[CPL];
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        lo_c[i] = 0.f;
        hi_c[i] = 0.f;
        if (active) {
          const int j = part * CPL + i;                   // chunk 0..15 of the row: half j >> 3, chunk j & 7
          const int phys = ((j & 7) + row) & 7;           // which 16 bytes of the line: rotated against bank conflicts
          const uint4 c = *reinterpret_cast<const uint4*>(xt + (j >> 3) * kDcXHalfBytes + row * 128 + phys * 16);
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&c.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&c.y));
          const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&c.z));
          const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&c.w));
          lo_c[i] = (f0.x + f0.y) + (f2.x + f2.y);
          hi_c[i] = (f1.x + f1.y) + (f3.x + f3.y);
        }
      }
#pragma unroll
      for (int w = 1; w < CPL; w <<= 1) {
#pragma unroll
        for (int i = 0; i < CPL; i += 2 * w) {
          lo_c[i] += lo_c[i + w];
          hi_c[i] += hi_c[i + w];
        }
      }
      float lo = lo_c[0], hi = hi_c[0];
#pragma unroll
      for (int off = 1; off < P; off <<= 1) {
        lo += __shfl_xor_sync(0xffffffffu, lo, off);
        hi += __shfl_xor_sync(0xffffffffu, hi, off);
      }
      if (active && part == 0) sums[s * MR + row] = make_float2(lo + hi, fmaf(1024.f, lo, 64.f * hi));
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_sums_full(s));
        mbar_arrive(bar_empty_tma(t));
      }
    }
    __syncwarp();
  } else {
    // ---------------------- unpack, then read accumulators back ---------------
    // Warp (quarter q, half h, group g): thread = column h*128 + 32q + lane of the tile.  The two groups take
    // the units in turn; a thread unpacks all 16 words of its column per unit it handles (64 tensor-memory
    // columns, four stores of 16) and, one unit of its own later, folds that unit's accumulator into acc[].
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y and the workspace belong to the previous kernel until here
    const int id = tid - 64;                  // 0..511
    const int dq_warp = id >> 5;              // 0..15
    const int lane_q = warp & 3;              // TMEM lane quarter this warp may touch
    const int idx = dq_warp >> 2;             // 0..3, each (quarter, idx) pair exactly once
    const int h = idx & 1, grp = idx >> 1;
    const int cl = h * 128 + lane_q * 32 + lane;            // column within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(lane_q * 32) << 16;
    const uint32_t raw_off = static_cast<uint32_t>(kDcRawOff + cl * 64);
    const uint32_t swz = static_cast<uint32_t>((cl >> 1) & 3);
    const int zcols = p.N >> 3;
    bool ok = true;
    int gs = 0, seg = 0;
    while (gs < my_units) {
      const long long u = u0 + gs;
      const int tile = static_cast<int>(u / nblk);
      const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * nblk);
      const int seg_units = min(nblk - kb0, my_units - gs);
      const int n0 = tile * kDcBN;
      const int n = n0 + cl;
      const bool nvalid = n < p.N;
      const uint32_t zsh = awq_slot_shift(static_cast<uint32_t>(n & 7));
      uint32_t sc = 0u, zw = 0u;
      int sz_group = -1;
      float acc[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[m] = 0.f;
      int pend = -1;                          // unit of this group whose accumulator is still in tensor memory
      float pend_s = 0.f, pend_z = 0.f;

      // acc[m] += s * (D[m] - H[m] - z * S[m]) for the pending unit
      auto fold_pending = [&]() {
        if (pend < 0) return;
        const int w = pend % NW, s = pend % NS;
        if (ok && !mbar_wait(bar_win_full(h, w), static_cast<uint32_t>(pend / NW) & 1u, abort_flag, 6)) ok = false;
        if (ok && !mbar_wait(bar_sums_full(s), static_cast<uint32_t>(pend / NS) & 1u, abort_flag, 9)) ok = false;
        if (ok) {
          tcgen05_fence_after();
          uint32_t v[MR];
          tmem_ld_row<MR>(tmem_base + lane_addr + static_cast<uint32_t>((w * 2 + h) * kDcMT), v);
          tcgen05_wait_ld();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_win_empty(h, w));
          const float nz = -pend_z;
#pragma unroll
          for (int m = 0; m < MR; ++m) {
            const float2 sh = sums[s * MR + m];            // same address in every lane: a broadcast
            acc[m] = fmaf(pend_s, fmaf(nz, sh.x, __uint_as_float(v[m]) - sh.y), acc[m]);
          }
        }
        pend = -1;
      };

      for (int j = 0; j < seg_units; ++j, ++gs) {
        if ((gs & 1) != grp) continue;                           // the other group's unit
        const int t = gs % NT, a = gs % NA;
        const uint32_t ph = static_cast<uint32_t>(gs / NT) & 1u, pha = static_cast<uint32_t>(gs / NA) & 1u;
        if (!sz_by_copy) {
          const int qgrp = ((kb0 + j) * kBlockK) / p.group_size;
          if (qgrp != sz_group) {
            sc = nvalid ? __ldg(p.scales + static_cast<size_t>(qgrp) * p.N + n) : 0u;
            zw = nvalid ? __ldg(p.qzeros + static_cast<size_t>(qgrp) * zcols + (n >> 3)) : 0u;
            sz_group = qgrp;
          }
        }
        if (ok && !mbar_wait(bar_full_tma(t), ph, abort_flag, 5)) ok = false;
        if (!ok) continue;
        const unsigned char* stage = base_ptr + t * kDcStageBytes;
        if (sz_by_copy) {
          // Columns beyond N read stale shared memory here; their lanes of the product are never stored.
          sc = reinterpret_cast<const uint16_t*>(stage + kDcSzOff)[cl];
          zw = reinterpret_cast<const uint32_t*>(stage + kDcSzOff + 512)[cl >> 3];
        }
        uint4 r[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          r[c] = *reinterpret_cast<const uint4*>(stage + raw_off + ((static_cast<uint32_t>(c) ^ swz) << 4));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty_tma(t));            // packed weights are in registers
        if (!mbar_wait(bar_a_empty(a), pha ^ 1u, abort_flag, 7)) { ok = false; continue; }
        tcgen05_fence_after();
        const uint32_t a_addr = tmem_base + lane_addr + static_cast<uint32_t>(kDcABase + a * 128 + h * 64);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t w4[4] = {r[c].x, r[c].y, r[c].z, r[c].w};
          uint32_t o[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t q4[4];
            unpack_codes(w4[i], q4);
            o[4 * i + 0] = q4[0]; o[4 * i + 1] = q4[1]; o[4 * i + 2] = q4[2]; o[4 * i + 3] = q4[3];
          }
          tcgen05_st_32x32b_x16(a_addr + static_cast<uint32_t>(c * 16), o);
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_a_full(a));
        // this group's previous unit: its MMAs were issued a whole unit of work ago
        fold_pending();
        pend = gs;
        pend_s = __half2float(__ushort_as_half(static_cast<unsigned short>(sc)));
        pend_z = small_uint_to_float((zw >> zsh) & 0xFu);
      }
      fold_pending();

      // ------------------------------ segment epilogue ------------------------
      // Group 1 hands its sums to group 0 through shared memory (double-buffered on the segment parity: the
      // barrier below keeps the groups at most one segment apart), group 0 finishes the tile.
      float* cb = comb + (seg & 1) * (MR * kDcBN);
      if (grp == 1) {
#pragma unroll
        for (int m = 0; m < MR; ++m) cb[m * kDcBN + cl] = acc[m];
      }
      unpack_warps_sync();
      // Contributors of this column tile: the CTAs that own its first and last unit, and all between.
      const long long tile_u0 = static_cast<long long>(tile) * nblk;
      const int c_first = stream_cta_of(tile_u0, U, G);
      const int c_last = stream_cta_of(tile_u0 + nblk - 1, U, G);
      const int nc = c_last - c_first + 1;
      const int slot = static_cast<int>(blockIdx.x) - c_first;
      const bool direct = (nc == 1);
      if (grp == 0) {
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          if (m < p.M) {                                   // warp-uniform
            const float val = acc[m] + cb[m * kDcBN + cl];
            // 32 lanes = 32 consecutive columns starting at a multiple of 32: 64 contiguous bytes of a row
            if (direct) epilogue_store_lane(p.y, p.epi, m, p.N, n, val, nvalid);
            else if (nvalid) __stcg(p.partial + (static_cast<size_t>(slot) * p.M + m) * p.N + n, val);
          }
        }
      }
      if (!direct) {
        __threadfence();
        unpack_warps_sync();
        if (id == 0) {
          const unsigned prev = atomicAdd(&p.counters[tile], 1u);
          const int last = (prev == static_cast<unsigned>(nc - 1));
          if (last) p.counters[tile] = 0u;   // every contributor has arrived: leave the counter clean
          s_last = last;
        }
        unpack_warps_sync();
        if (s_last) {
          __threadfence();
          // The last contributor adds the nc slots in CTA order, which is k order.
          const int ncols = min(kDcBN, p.N - n0);
          const int pairs = ncols >> 1;
          const size_t slot_stride = static_cast<size_t>(p.M) * p.N;
          for (int i = id; i < p.M * pairs; i += kDcUnpackThreads) {
            const int row = i / pairs;
            const int col = n0 + 2 * (i - row * pairs);
            const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
            float2 sum = __ldcg(reinterpret_cast<const float2*>(src));
            for (int s = 1; s < nc; ++s) {
              const float2 v = __ldcg(reinterpret_cast<const float2*>(src + s * slot_stride));
              sum.x += v.x;
              sum.y += v.y;
            }
            epilogue_store_pair(p.y, p.epi, row, p.N, col, sum.x, sum.y);
          }
        }
        unpack_warps_sync();   // s_last is rewritten by the next straddling segment
      }
      ++seg;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, 0x300u | static_cast<unsigned>(s_abort));
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static int decode_grid(int sm_count, long long units) {
  return static_cast<int>(units < sm_count ? units : sm_count);
}

// Largest number of CTAs that share one column tile (= partial slots needed).
static int decode_slots(int K, int N, int sm_count) {
  const int nblk = K / kBlockK, ntiles = (N + kDcBN - 1) / kDcBN;
  const long long U = static_cast<long long>(ntiles) * nblk;
  const long long G = decode_grid(sm_count, U);
  int worst = 1;
  for (int t = 0; t < ntiles; ++t) {
    const long long a = static_cast<long long>(t) * nblk;
    const int nc = stream_cta_of(a + nblk - 1, U, G) - stream_cta_of(a, U, G) + 1;
    if (nc > worst) worst = nc;
  }
  return worst;
}

static size_t decode_counter_bytes() { return kGemvMaxCounters * sizeof(unsigned); }

size_t decode_workspace_bytes(int M, int K, int N, int sm_count) {
  if (M < 1 || K < kBlockK || N < 8) return 0;
  const int slots = decode_slots(K, N, sm_count);
  return decode_counter_bytes() + (slots > 1 ? static_cast<size_t>(slots) * M * N * sizeof(float) : 0);
}

template <int MR>
static int launch_decode(const void* x, const void* packed, DcParams p, int grid, EncodeTiledFn encode,
                         cudaStream_t stream, bool overlap_previous, int max_smem_optin) {
  using Cfg = DcCfg<MR>;
  if (Cfg::kSmemBytes > max_smem_optin) return AWQ_B200_ERR_TOO_LARGE;
  CUtensorMap mx, mw;
  {
    // rows beyond M are outside the tensor: the copy fills them with zeros
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.K) * 2};
    const cuuint32_t box[2] = {64, kDcMT};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  {
    // packed weights as [k block][column][64 bytes]; one box = one unit = 256 columns x 64 bytes
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.K / kBlockK)};
    const cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(p.N) * 64};
    const cuuint32_t box[3] = {64, kDcBN, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(packed), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  AWQ_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kDcThreads);
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
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_kernel<MR>, mx, mw, p));
  return AWQ_B200_OK;
}

int decode_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                    void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream, unsigned flags) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size)) return st;
  if (M < 1 || M > kDcMT) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) || !aligned16(y))
    return AWQ_B200_ERR_ALIGN;
  if (int st = check_epilogue(epi, N)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;
  EncodeTiledFn encode;
  if (int st = get_encode(&encode)) return st;
  const int ntiles = (N + kDcBN - 1) / kDcBN;
  if (ntiles > kGemvMaxCounters - 1) return AWQ_B200_ERR_TOO_LARGE;
  if (!workspace || workspace_bytes < decode_workspace_bytes(M, K, N, di.sm_count)) return AWQ_B200_ERR_WORKSPACE;
  if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
  DcParams p;
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.epi = epi;
  p.y = static_cast<uint16_t*>(y);
  p.counters = static_cast<unsigned*>(workspace);
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + decode_counter_bytes());
  p.status = static_cast<unsigned*>(workspace) + (kGemvMaxCounters - 1);
  p.M = M; p.K = K; p.N = N;
  p.group_size = group_size;
  p.ntiles = ntiles;
  p.nblk = K / kBlockK;
  p.units = static_cast<long long>(ntiles) * p.nblk;
  const int grid = decode_grid(di.sm_count, p.units);
  const bool overlap = (flags & AWQ_B200_OVERLAP_PREVIOUS) != 0;
  if (M <= 1) return launch_decode<1>(x, packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  if (M <= 2) return launch_decode<2>(x, packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  if (M <= 4) return launch_decode<4>(x, packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  if (M <= 8) return launch_decode<8>(x, packed, p, grid, encode, stream, overlap, di.max_smem_optin);
  return launch_decode<16>(x, packed, p, grid, encode, stream, overlap, di.max_smem_optin);
}

}  // namespace awq

extern "C" {

size_t awq_b200_decode_workspace_bytes(int M, int K, int N) {
  awq::DeviceInfo di;
  int sm = 148;
  if (awq::device_info(&di) == AWQ_B200_OK) sm = di.sm_count;
  return awq::decode_workspace_bytes(M, K, N, sm);
}

int awq_b200_decode(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                    void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                    awq_b200_stream_t stream, unsigned flags) {
  return awq::decode_dispatch(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y,
                              M, K, N, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), flags);
}

}  // extern "C"
