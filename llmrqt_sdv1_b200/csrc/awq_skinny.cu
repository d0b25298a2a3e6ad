// W4A16 linear for few activation rows (1 <= M <= 64) on the tcgen05 path: split-K over a persistent,
// evenly balanced stream of work units, with the weights as the tensor-memory A operand.
//
//   Y^T[n, m] = sum_k W^T[n, k] * X^T[k, m]
//
// The arithmetic is that of the weights-in-tensor-memory GEMM (awq_wtm.cu): dequant warps turn
// packed nibbles into the exact reference fp16 weight in registers and write it into tensor memory
// (lane = output column, two consecutive k per 32-bit column); tcgen05.mma takes A = W^T from
// tensor memory, B = the activation rows (K-major, 128-byte swizzle, staged by TMA) from shared
// memory, and accumulates in fp32 in tensor memory over the whole k range of a segment.  No
// per-block rescaling, no mma.sync fragments: per packed word the SM only runs the unpack itself.
//
// Work distribution (what makes this the decode kernel for large matrices):
//   unit      = one 128-k block of one tile of 256 output columns: 16 KiB of packed weights.
//   CTA b     = units [b*U/G, (b+1)*U/G) of the flattened (column tile, k block) sequence, G = one CTA
//               per SM; one copy pipeline per CTA runs through all of them without draining.
//   segment   = the units of one column tile inside one CTA.  A tile that lies inside one CTA is
//               written straight to y; one that straddles CTAs is written as fp32 partials, one slot
//               per contributing CTA, and the last contributor to arrive adds the slots in CTA order
//               (= k order).  Deterministic, and a row's bits do not depend on M: the partition
//               depends on (K, N) only and the MMA N extent does not change how an element is summed.
//
// Warps: 0 and 18 copy producers (even / odd units), 1 and 19 MMA issuers (low / high 128 columns),
// 2..17 dequantise (two groups of eight that take the units in turn) and, at the end of a segment,
// drain the accumulators.
// TMEM columns: [0, MT) and [MT, 2MT) accumulators of the two halves, then the A ring (128 columns
// per unit: 64 per half).  Every mbarrier wait is bounded (see awq_ptx.cuh).
#include "awq_gemv_common.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kSkDequantWarps = 16;
constexpr int kSkDequantThreads = kSkDequantWarps * 32;
constexpr int kSkThreads = 64 + kSkDequantThreads + 64;
constexpr int kSkProducer2Warp = 18, kSkIssuer2Warp = 19;
constexpr int kSkBN = 256;                       // output columns per tile
constexpr int kSkRawBytes = kSkBN * 64;          // one unit of packed weights: [256 columns][64 bytes], 64-byte swizzle

template <int MT> struct SkCfg {
  static_assert(MT == 16 || MT == 32 || MT == 64, "activation rows per tile");
  static constexpr int kXHalfBytes = MT * 128;                       // MT rows x 64 k
  static constexpr int kXBytes = 2 * kXHalfBytes;
  static constexpr int kXBytesPadded = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kRawOff = kXBytesPadded;
  static constexpr int kSzOff = kRawOff + kSkRawBytes;               // 256 fp16 scales, then 32 qzeros words
  static constexpr int kStageBytes = kSzOff + 1024;
  static constexpr int kStagesRaw = 200 * 1024 / kStageBytes;
  static constexpr int kStages = kStagesRaw >= 8 ? 8 : (kStagesRaw & ~1);
  static constexpr int kABase = 2 * MT;
  static constexpr int kAStages = (512 - 2 * MT) / 128;              // 3
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kStages >= 4 && kStages % 2 == 0, "two producers alternate over an even ring");
  static_assert(kAStages >= 2, "need a double-buffered A ring");
};

struct SkParams {
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

__device__ __forceinline__ void dequant_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kSkDequantThreads) : "memory");
}

template <int MT>
__global__ void __launch_bounds__(kSkThreads, 1)
skinny_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const SkParams p) {
  using Cfg = SkCfg<MT>;
  constexpr int NT = Cfg::kStages, NA = Cfg::kAStages;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ uint32_t s_tmem_base;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  auto stage_addr = [&](int t) { return base + t * Cfg::kStageBytes; };
  const uint32_t bar_base = base + NT * Cfg::kStageBytes;
  auto bar_full_tma = [&](int t) { return bar_base + 8u * t; };
  auto bar_empty_tma = [&](int t) { return bar_base + 8u * (NT + t); };    // 8 dequant warps + 2 MMA commits
  auto bar_a_full = [&](int a) { return bar_base + 8u * (2 * NT + a); };
  auto bar_a_empty = [&](int a) { return bar_base + 8u * (2 * NT + NA + a); };
  const uint32_t bar_acc_full = bar_base + 8u * (2 * NT + 2 * NA);
  const uint32_t bar_acc_empty = bar_base + 8u * (2 * NT + 2 * NA + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    s_abort = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_full_tma(t), 1);
      mbar_init(bar_empty_tma(t), kSkDequantWarps / 2 + 2);
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(bar_a_full(a), kSkDequantWarps / 2);
      mbar_init(bar_a_empty(a), 2);
    }
    mbar_init(bar_acc_full, 2);
    mbar_init(bar_acc_empty, kSkDequantWarps);
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
  constexpr uint32_t kIdesc = make_f16_idesc(128, MT);
  // Bulk copies need 16-byte aligned, 16-byte sized row segments of scales and qzeros: N % 32 == 0.  Groups
  // of 32 or 64 put several scale rows into one 128-k unit: those are read per thread instead.
  const bool sz_by_copy = (p.N & 31) == 0 && p.group_size >= kBlockK;
  const bool small_groups = p.group_size < kBlockK;

  if (warp == 0 || warp == kSkProducer2Warp) {
    // ------------------------------ copy producers ----------------------------
    // Warp-uniform loops; lanes 0..4 each issue one of a unit's five copies.  The weight-side copies
    // of the first ring fill are constant data and start before the wait on the previous kernel of
    // the stream; the activation boxes follow it.
    const int my_parity = warp == 0 ? 0 : 1;
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    // This producer's cursor: unit u0 + my_parity, then every second unit.
    int tile, kb;
    {
      const long long u = u0 + my_parity;
      tile = static_cast<int>(u / nblk);
      kb = static_cast<int>(u - static_cast<long long>(tile) * nblk);
    }
    const int group_blocks = p.group_size >= kBlockK ? p.group_size / kBlockK : 1;   // only used with sz_by_copy
    auto advance = [&]() {
      kb += 2;
      while (kb >= nblk) { kb -= nblk; ++tile; }
    };
    auto issue = [&](int gs, int tile_, int kb_, bool weights, bool activations) {
      const int n0 = tile_ * kSkBN;
      const int ncols = min(kSkBN, p.N - n0);
      const int t = gs % NT;
      const uint32_t bar = bar_full_tma(t);
      const uint32_t dst = stage_addr(t);
      if (weights) {
        if (lane == 0)
          mbar_expect_tx(bar, Cfg::kXBytes + kSkRawBytes + (sz_by_copy ? ncols * 2 + ncols / 2 : 0));
        if (lane == 2) tma_load_3d(dst + Cfg::kRawOff, &map_w, 0, n0, kb_, bar);
        if (sz_by_copy && (lane == 3 || lane == 4)) {
          const int grp = group_blocks == 1 ? kb_ : kb_ / group_blocks;
          if (lane == 3) bulk_load(dst + Cfg::kSzOff, p.scales + static_cast<size_t>(grp) * p.N + n0, ncols * 2, bar);
          else bulk_load(dst + Cfg::kSzOff + 512, p.qzeros + static_cast<size_t>(grp) * (p.N >> 3) + (n0 >> 3), ncols / 2, bar);
        }
      }
      if (activations && lane < 2) tma_load_2d(dst + lane * Cfg::kXHalfBytes, &map_x, kb_ * kBlockK + lane * 64, 0, bar);
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
    // Do not leave while a copy of this warp may still be writing shared memory: wait (bounded) for
    // the last ring's worth of its units to land.
    const int issued_end = next < my_units ? next : my_units;
    for (int gs = my_parity; gs < issued_end; gs += 2)
      if (gs + NT >= issued_end) mbar_wait_timed(bar_full_tma(gs % NT), static_cast<uint32_t>(gs / NT) & 1u);
    __syncwarp();
  } else if (warp == 1 || warp == kSkIssuer2Warp) {
    // ------------------------------ MMA issuers --------------------------------
    // One warp per 128-column half; warp-uniform loop, one elected lane issues.
    const int h = warp == 1 ? 0 : 1;
    int seg = 0;
    bool ok = true;
    int gs = 0, t = 0, a = 0;
    uint32_t ph = 0, pha = 0;
    while (gs < my_units && ok) {
      const long long u = u0 + gs;
      const int tile = static_cast<int>(u / nblk);
      const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * nblk);
      const int seg_units = min(nblk - kb0, my_units - gs);
      if (!mbar_wait(bar_acc_empty, (static_cast<uint32_t>(seg) & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
      tcgen05_fence_after();
      for (int j = 0; j < seg_units; ++j, ++gs) {
        if (!mbar_wait(bar_full_tma(t), ph, abort_flag, 3)) { ok = false; break; }
        if (!mbar_wait(bar_a_full(a), pha, abort_flag, 4)) { ok = false; break; }
        tcgen05_fence_after();
        // eight k-steps into this half's accumulator, then: activations of this unit consumed, A slot reusable
        tcgen05_mma_f16_ts_k8_commit2_warp(tmem_base + h * MT,
                                           tmem_base + static_cast<uint32_t>(Cfg::kABase + a * 128 + h * 64),
                                           make_sw128_desc(stage_addr(t)), 32u >> 4, Cfg::kXHalfBytes >> 4, kIdesc,
                                           j != 0 ? 1u : 0u, bar_empty_tma(t), bar_a_empty(a));
        if (++t == NT) { t = 0; ph ^= 1u; }
        if (++a == NA) { a = 0; pha ^= 1u; }
      }
      if (ok) tcgen05_commit_warp(bar_acc_full);
      ++seg;
    }
    __syncwarp();
  } else {
    // ---------------------- dequantise, then drain accumulators ---------------
    // Warp (quarter q, half h, group g): thread = column h*128 + 32q + lane.  The two groups take the
    // units in turn, so that one group's latency chain (wait, unpack, tensor-memory store, arrive)
    // overlaps the other's; a thread unpacks all 16 words of its column per unit it handles: 64
    // tensor-memory columns, four stores of 16.
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y and the workspace belong to the previous kernel until here
    const int id = tid - 64;                  // 0..511
    const int dq_warp = id >> 5;              // 0..15
    const int lane_q = warp & 3;              // TMEM lane quarter this warp may touch
    const int idx = dq_warp >> 2;             // 0..3, each (quarter, idx) pair exactly once
    const int h = idx & 1, grp = idx >> 1;
    const int cl = h * 128 + lane_q * 32 + lane;            // column within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(lane_q * 32) << 16;
    const uint32_t raw_off = static_cast<uint32_t>(Cfg::kRawOff + cl * 64);
    const uint32_t swz = static_cast<uint32_t>((cl >> 1) & 3);
    const int zcols = p.N >> 3;
    // epilogue role: half e_h, rows [e_part * MT/2, +MT/2)
    const int e_h = h, e_part = grp;
    bool ok = true;
    int gs = 0, seg = 0;
    while (gs < my_units) {
      const long long u = u0 + gs;
      const int tile = static_cast<int>(u / nblk);
      const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * nblk);
      const int seg_units = min(nblk - kb0, my_units - gs);
      const int n0 = tile * kSkBN;
      const int n = n0 + cl;
      const bool nvalid = n < p.N;
      const uint32_t zsh = awq_slot_shift(static_cast<uint32_t>(n & 7));
      uint32_t sc = 0u, zw = 0u;
      int sz_group = -1;

      for (int j = 0; j < seg_units; ++j, ++gs) {
        if ((gs & 1) != grp) continue;                           // the other group's unit
        const int t = gs % NT, a = gs % NA;
        const uint32_t ph = static_cast<uint32_t>(gs / NT) & 1u, pha = static_cast<uint32_t>(gs / NA) & 1u;
        uint32_t sc_sub[4] = {0u, 0u, 0u, 0u}, zw_sub[4] = {0u, 0u, 0u, 0u};   // per 32 k of the unit (small groups)
        if (small_groups) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int qgrp = ((kb0 + j) * kBlockK + 32 * c) / p.group_size;
            if (c > 0 && qgrp == ((kb0 + j) * kBlockK + 32 * (c - 1)) / p.group_size) {
              sc_sub[c] = sc_sub[c - 1];
              zw_sub[c] = zw_sub[c - 1];
            } else {
              sc_sub[c] = nvalid ? __ldg(p.scales + static_cast<size_t>(qgrp) * p.N + n) : 0u;
              zw_sub[c] = nvalid ? __ldg(p.qzeros + static_cast<size_t>(qgrp) * zcols + (n >> 3)) : 0u;
            }
          }
        } else if (!sz_by_copy) {
          const int qgrp = ((kb0 + j) * kBlockK) / p.group_size;
          if (qgrp != sz_group) {
            sc = nvalid ? __ldg(p.scales + static_cast<size_t>(qgrp) * p.N + n) : 0u;
            zw = nvalid ? __ldg(p.qzeros + static_cast<size_t>(qgrp) * zcols + (n >> 3)) : 0u;
            sz_group = qgrp;
          }
        }
        if (ok && !mbar_wait(bar_full_tma(t), ph, abort_flag, 5)) ok = false;
        if (!ok) continue;
        const unsigned char* stage = base_ptr + t * Cfg::kStageBytes;
        if (sz_by_copy) {
          // Columns beyond N read stale shared memory here; their lanes of the product are never stored.
          sc = reinterpret_cast<const uint16_t*>(stage + Cfg::kSzOff)[cl];
          zw = reinterpret_cast<const uint32_t*>(stage + Cfg::kSzOff + 512)[cl >> 3];
        }
        uint4 r[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          r[c] = *reinterpret_cast<const uint4*>(stage + raw_off + ((static_cast<uint32_t>(c) ^ swz) << 4));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty_tma(t));            // packed weights are in registers
        if (!mbar_wait(bar_a_empty(a), pha ^ 1u, abort_flag, 7)) { ok = false; continue; }
        tcgen05_fence_after();
        ZeroPair zp = make_zero_pair((zw >> zsh) & 0xFu);
        uint32_t s2 = sc * 0x00010001u;
        const uint32_t a_addr = tmem_base + lane_addr + static_cast<uint32_t>(Cfg::kABase + a * 128 + h * 64);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (small_groups) {                                    // warp-uniform
            zp = make_zero_pair((zw_sub[c] >> zsh) & 0xFu);
            s2 = sc_sub[c] * 0x00010001u;
          }
          const uint32_t w[4] = {r[c].x, r[c].y, r[c].z, r[c].w};
          uint32_t o[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t q4[4];
            dequant_word(w[i], zp, s2, q4);
            o[4 * i + 0] = q4[0]; o[4 * i + 1] = q4[1]; o[4 * i + 2] = q4[2]; o[4 * i + 3] = q4[3];
          }
          tcgen05_st_32x32b_x16(a_addr + static_cast<uint32_t>(c * 16), o);
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_a_full(a));
      }

      // ------------------------------ segment epilogue ------------------------
      // Contributors of this column tile: the CTAs that own its first and last unit, and all between.
      const long long tile_u0 = static_cast<long long>(tile) * nblk;
      const int c_first = stream_cta_of(tile_u0, U, G);
      const int c_last = stream_cta_of(tile_u0 + nblk - 1, U, G);
      const int nc = c_last - c_first + 1;
      const int slot = static_cast<int>(blockIdx.x) - c_first;
      const bool direct = (nc == 1);
      if (ok && !mbar_wait(bar_acc_full, static_cast<uint32_t>(seg) & 1u, abort_flag, 6)) ok = false;
      if (ok) {
        tcgen05_fence_after();
        constexpr int kChunksPerPart = MT / 16;          // chunks of 8 activation rows per warp
#pragma unroll 1
        for (int ch = e_part * kChunksPerPart; ch < (e_part + 1) * kChunksPerPart; ++ch) {
          if (ch * 8 >= p.M) break;                      // rows beyond M are padding (warp-uniform)
          uint32_t v[8];
          asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                       : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                       : "r"(tmem_base + lane_addr + static_cast<uint32_t>(e_h * MT + ch * 8))
                       : "memory");
          tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = ch * 8 + i;
            if (m < p.M) {                               // warp-uniform
              const float val = __uint_as_float(v[i]);
              // 32 lanes = 32 consecutive columns starting at a multiple of 32: 64 contiguous bytes of a row
              if (direct) epilogue_store_lane(p.y, p.epi, m, p.N, n, val, nvalid);
              else if (nvalid) __stcg(p.partial + (static_cast<size_t>(slot) * p.M + m) * p.N + n, val);
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty);
      }
      if (!direct) {
        __threadfence();
        dequant_warps_sync();
        if (id == 0) {
          const unsigned prev = atomicAdd(&p.counters[tile], 1u);
          const int last = (prev == static_cast<unsigned>(nc - 1));
          if (last) p.counters[tile] = 0u;   // every contributor has arrived: leave the counter clean
          s_last = last;
        }
        dequant_warps_sync();
        if (s_last) {
          __threadfence();
          // The last contributor adds the nc slots in CTA order, which is k order.
          const int ncols = min(kSkBN, p.N - n0);
          const int pairs = ncols >> 1;
          const size_t slot_stride = static_cast<size_t>(p.M) * p.N;
          for (int i = id; i < p.M * pairs; i += kSkDequantThreads) {
            const int row = i / pairs;
            const int col = n0 + 2 * (i - row * pairs);
            const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
            const float2 sum = sum_partial_slots(src, slot_stride, nc);
            epilogue_store_pair(p.y, p.epi, row, p.N, col, sum.x, sum.y);
          }
        }
        dequant_warps_sync();   // s_last is rewritten by the next straddling segment
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
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, 0x200u | static_cast<unsigned>(s_abort));
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static int skinny_grid(int sm_count, long long units) {
  return static_cast<int>(units < sm_count ? units : sm_count);
}

// Largest number of CTAs that share one column tile (= partial slots needed).
static int skinny_slots(int K, int N, int sm_count) {
  const int nblk = K / kBlockK, ntiles = (N + kSkBN - 1) / kSkBN;
  const long long U = static_cast<long long>(ntiles) * nblk;
  const long long G = skinny_grid(sm_count, U);
  int worst = 1;
  for (int t = 0; t < ntiles; ++t) {
    const long long a = static_cast<long long>(t) * nblk;
    const int nc = stream_cta_of(a + nblk - 1, U, G) - stream_cta_of(a, U, G) + 1;
    if (nc > worst) worst = nc;
  }
  return worst;
}

static size_t skinny_counter_bytes() { return kGemvMaxCounters * sizeof(unsigned); }

size_t skinny_workspace_bytes(int M, int K, int N, int sm_count) {
  if (M < 1 || K < kBlockK || N < 8) return 0;
  const int slots = skinny_slots(K, N, sm_count);
  return skinny_counter_bytes() + (slots > 1 ? static_cast<size_t>(slots) * M * N * sizeof(float) : 0);
}

template <int MT>
static int launch_skinny(const void* x, const void* packed, SkParams p, int grid, EncodeTiledFn encode,
                         cudaStream_t stream, bool overlap_previous) {
  using Cfg = SkCfg<MT>;
  CUtensorMap mx, mw;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.K) * 2};
    const cuuint32_t box[2] = {64, MT};
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
    const cuuint32_t box[3] = {64, kSkBN, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(packed), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  AWQ_CUDA_TRY(cudaFuncSetAttribute(skinny_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kSkThreads);
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
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, skinny_kernel<MT>, mx, mw, p));
  return AWQ_B200_OK;
}

int skinny_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                    void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream, unsigned flags) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size, true)) return st;
  if (M < 1 || M > 64) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) || !aligned16(y))
    return AWQ_B200_ERR_ALIGN;
  if (int st = check_epilogue(epi, N)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;
  EncodeTiledFn encode;
  if (int st = get_encode(&encode)) return st;
  const int ntiles = (N + kSkBN - 1) / kSkBN;
  if (ntiles > kGemvMaxCounters - 1) return AWQ_B200_ERR_TOO_LARGE;
  if (!workspace || workspace_bytes < skinny_workspace_bytes(M, K, N, di.sm_count)) return AWQ_B200_ERR_WORKSPACE;
  if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
  SkParams p;
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.epi = epi;
  p.y = static_cast<uint16_t*>(y);
  p.counters = static_cast<unsigned*>(workspace);
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + skinny_counter_bytes());
  p.status = static_cast<unsigned*>(workspace) + (kGemvMaxCounters - 1);
  p.M = M; p.K = K; p.N = N;
  p.group_size = group_size;
  p.ntiles = ntiles;
  p.nblk = K / kBlockK;
  p.units = static_cast<long long>(ntiles) * p.nblk;
  const int grid = skinny_grid(di.sm_count, p.units);
  const bool overlap = (flags & AWQ_B200_OVERLAP_PREVIOUS) != 0;
  if (M <= 16) return launch_skinny<16>(x, packed, p, grid, encode, stream, overlap);
  if (M <= 32) return launch_skinny<32>(x, packed, p, grid, encode, stream, overlap);
  return launch_skinny<64>(x, packed, p, grid, encode, stream, overlap);
}

}  // namespace awq

extern "C" {

size_t awq_b200_skinny_workspace_bytes(int M, int K, int N) {
  awq::DeviceInfo di;
  int sm = 148;
  if (awq::device_info(&di) == AWQ_B200_OK) sm = di.sm_count;
  return awq::skinny_workspace_bytes(M, K, N, sm);
}

int awq_b200_skinny(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                    void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                    awq_b200_stream_t stream, unsigned flags) {
  return awq::skinny_dispatch(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace, workspace_bytes,
                              static_cast<cudaStream_t>(stream), flags);
}

}  // extern "C"
