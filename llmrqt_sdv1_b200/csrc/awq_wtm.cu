// W4A16 GEMM with the weights as the TMEM-resident A operand ("weights in tensor memory").
//
//   Y^T[n, m] = sum_k W^T[n, k] * X^T[k, m]
//
// The 16 dequant warps turn packed nibbles into the exact reference fp16 weight in registers and
// write it straight into tensor memory (tcgen05.st): lane = output column n, two consecutive k per
// 32-bit TMEM column.  tcgen05.mma then takes A = W^T from tensor memory and B = X (K-major rows
// of the activations, staged by TMA with the 128-byte swizzle) from shared memory, with fp32
// accumulators in tensor memory as well.  Compared with staging the dequantised weights in shared
// memory this removes their shared-memory write and re-read, which is what bounds that variant.
//
// CTA tile: 256 output columns (two 128-lane halves) x MT activation rows, 64-k stages:
//   warp 0      TMA producer: X tile [MT x 64] and the packed weights [256 columns x 32 bytes, 32-byte swizzle]
//   warp 1      TMEM allocation, tcgen05.mma issue (M=128, N=MT, K=16), one thread
//   warps 2-17  dequantise (4 words = 32 k of one column per thread and stage), then drain the
//               accumulators: thread = column n, it reads MT values of its lane and stores Y[m, n]
// TMEM columns: [0, MT) and [MT, 2MT) accumulators of the two halves, then the A ring
// (32 columns per half and stage).  Every mbarrier wait is bounded (see awq_ptx.cuh).
#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kWtDequantThreads = 512;
// warp 0 and warp 18: copy producers (even and odd k-stages); warp 1: MMA issuer; warps 2..17: dequantise + epilogue
constexpr int kWtProducer2Warp = 2 + kWtDequantThreads / 32;
constexpr int kWtThreads = 64 + kWtDequantThreads + 32;
constexpr int kWtBN = 256;       // output columns per CTA tile
constexpr int kWtBK = 64;
constexpr int kWtRawBytes = kWtBN * (kWtBK / 2);   // 8 KiB: [256 columns][32 bytes], 32-byte swizzle

template <int MT> struct WtCfg {
  static_assert(MT % 16 == 0 && MT >= 16 && MT <= 192, "the MMA N extent");
  static constexpr int kXBytes = MT * kWtBK * 2;                 // MT rows x 128 bytes
  static constexpr int kXBytesPadded = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kSzOff = kXBytesPadded + kWtRawBytes;         // 256 fp16 scales, then 32 qzeros words
  static constexpr int kStageBytes = kXBytesPadded + kWtRawBytes + 1024;
  static constexpr int kStages = (200 * 1024 / kStageBytes) < 8 ? (200 * 1024 / kStageBytes) : 8;
  static constexpr int kAStages = (512 - 2 * MT) / 64 < 4 ? (512 - 2 * MT) / 64 : 4;   // A ring depth (stages)
  static constexpr int kABase = 2 * MT;                          // first TMEM column of the A ring
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kAStages >= 2, "need a double-buffered A ring");
  // The 16 dequant warps work in kGroups groups that take the k-stages in turn, so that a warp's
  // latency chain (wait, unpack, tensor-memory store, arrive) overlaps the other groups' work.
  static constexpr int kGroups = kAStages < 4 ? kAStages : 4;
  static constexpr int kGroupWarps = 16 / kGroups;
};

struct WtParams {
  const uint16_t* scales;
  const uint32_t* qzeros;
  Epilogue epi;
  uint16_t* y;
  unsigned* status;
  float* partial;        // tail split only: two fp32 tiles [MT][256] per CTA
  int M, K, N;
  int group_size;
  int mtiles, ntiles;
  int tail_split;        // 1: the tiles of the last, partial wave are cut along k and shared by all CTAs
};

// What a CTA works on, in order: its tile of every full wave, then its share of the last wave.  With
// the tail split the tiles left over after the full waves (fewer than there are CTAs) are flattened
// into (tile, 64-k stage) units and every CTA takes an equal, contiguous share; a share touches at
// most two tiles.  A tile finished by several CTAs goes through fp32 partial tiles in the workspace
// (slot 2*b + 0/1 for CTA b's first / second tail item); a small second kernel adds them in CTA (= k)
// order and writes y, so no CTA ever waits for another.
struct WtItem {
  int tile;        // global tile index
  int ks0, ks1;    // 64-k stages [ks0, ks1)
  int tail;        // index among the tail tiles, or -1 for a tile of a full wave
};
struct WtCursor {
  int b, G, nks, full_rounds, tail_tiles, r;
  long long u, u_end, Ut;
  __device__ void init(int b_, int G_, int nks_, int num_tiles, int tail_split) {
    b = b_; G = G_; nks = nks_; r = 0;
    full_rounds = tail_split ? num_tiles / G : (num_tiles + G - 1) / G;
    tail_tiles = tail_split ? num_tiles - full_rounds * G : 0;
    total_tiles = num_tiles;
    Ut = static_cast<long long>(tail_tiles) * nks;
    u = b * Ut / G;
    u_end = (b + 1) * Ut / G;
  }
  int total_tiles;
  __device__ bool next(WtItem* w) {
    while (r < full_rounds) {
      const int tile = r * G + b;
      ++r;
      if (tile < total_tiles) { *w = WtItem{tile, 0, nks, -1}; return true; }
    }
    if (u < u_end) {
      const int tt = static_cast<int>(u / nks);
      const int k0 = static_cast<int>(u - static_cast<long long>(tt) * nks);
      const int len = static_cast<int>(min(static_cast<long long>(nks - k0), u_end - u));
      *w = WtItem{full_rounds * G + tt, k0, k0 + len, tt};
      u += len;
      return true;
    }
    return false;
  }
};


template <int MT>
__global__ void __launch_bounds__(kWtThreads, 1)
wtm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const WtParams p) {
  using Cfg = WtCfg<MT>;
  constexpr int NT = Cfg::kStages, NA = Cfg::kAStages;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem_base;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  auto x_addr = [&](int t) { return base + t * Cfg::kStageBytes; };
  auto raw_addr = [&](int t) { return base + t * Cfg::kStageBytes + Cfg::kXBytesPadded; };
  const uint32_t bar_base = base + NT * Cfg::kStageBytes;
  auto bar_full_tma = [&](int t) { return bar_base + 8u * t; };
  auto bar_empty_tma = [&](int t) { return bar_base + 8u * (NT + t); };    // MMA commit + 16 dequant warps
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
      mbar_init(bar_empty_tma(t), 1 + Cfg::kGroupWarps);
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(bar_a_full(a), Cfg::kGroupWarps);
      mbar_init(bar_a_empty(a), 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, kWtDequantThreads / 32);
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
  const int nks = p.K / kWtBK;
  const int num_tiles = p.mtiles * p.ntiles;
  constexpr uint32_t kIdesc = make_f16_idesc(128, MT);
  // Bulk copies need 16-byte aligned, 16-byte sized row segments of scales and qzeros: N % 32 == 0.
  // Scales and zero words ride in the stage by bulk copy when their row segments are 16-byte aligned and sized
  // (N % 32 == 0) and a 64-k stage lies within one quantisation group; groups of 32 are read per thread.
  const bool sz_by_copy = (p.N & 31) == 0 && p.group_size >= kWtBK;
  const bool half_stage_groups = p.group_size < kWtBK;

  if (warp == 0 || warp == kWtProducer2Warp) {
    // ------------------------------ TMA producers -----------------------------
    // Two warps take the k-stages alternately: one warp's issue chain (wait, expect, three copy
    // instructions) is longer than the time a small-MT stage takes to consume.
    static_assert(NT % 2 == 0, "the two producers alternate over an even ring");
    const uint32_t my_parity = warp == 0 ? 0u : 1u;
    // Warp-uniform loop; lanes 0, 1, 3 and 4 each issue one of the stage's four copies, so that a stage costs
    // three predicated instructions rather than a serial chain in one thread.
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    const int stages_per_group = p.group_size >= kWtBK ? p.group_size / kWtBK : 1;   // only used with sz_by_copy
    uint32_t it = 0;
    int t = 0;
    uint32_t ph = 0;
    bool ok = true;
    WtCursor cur;
    cur.init(blockIdx.x, gridDim.x, nks, num_tiles, p.tail_split);
    WtItem w;
    while (ok && cur.next(&w)) {
      int tile_m, tile_n;
      tile_coords(w.tile, p.mtiles, p.ntiles, &tile_m, &tile_n);
      const int m0 = tile_m * MT;
      const int n0 = tile_n * kWtBN;
      const int ncols = min(kWtBN, p.N - n0);
      const uint32_t tx = Cfg::kXBytes + kWtRawBytes + (sz_by_copy ? ncols * 2 + ncols / 2 : 0);
      int grp = w.ks0 / stages_per_group, left = stages_per_group - (w.ks0 - grp * stages_per_group);
      // lane 3 copies the scales row segment, lane 4 the zero words
      const unsigned char* sz_src = (lane == 3) ? reinterpret_cast<const unsigned char*>(p.scales + n0)
                                                : reinterpret_cast<const unsigned char*>(p.qzeros + (n0 >> 3));
      const size_t sz_step = (lane == 3) ? static_cast<size_t>(p.N) * 2 : static_cast<size_t>(p.N >> 3) * 4;
      const uint32_t sz_bytes = (lane == 3) ? ncols * 2 : ncols / 2;
      const uint32_t sz_dst = Cfg::kSzOff + (lane == 3 ? 0 : 512);
      for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
        if ((it & 1u) == my_parity) {
          if (!mbar_wait(bar_empty_tma(t), ph ^ 1u, abort_flag, 1)) { ok = false; break; }
          const uint32_t bar = bar_full_tma(t);
          if (lane == 0) {
            mbar_expect_tx(bar, tx);
            tma_load_2d(x_addr(t), &map_x, ks * kWtBK, m0, bar);
          }
          // packed weights of this 64-k stage: bytes [32*(ks&1), +32) of each column's 64 per 128-k block, one
          // 32-byte row per column; the 32-byte swizzle makes the per-column 16-byte reads conflict-free
          if (lane == 1) tma_load_3d(raw_addr(t), &map_w, (ks & 1) * 32, n0, ks >> 1, bar);
          // scales and zero words of this stage's quantisation group ride in the same stage
          if (sz_by_copy && (lane == 3 || lane == 4))
            bulk_load(x_addr(t) + sz_dst, sz_src + static_cast<size_t>(grp) * sz_step, sz_bytes, bar);
        }
        if (--left == 0) { left = stages_per_group; ++grp; }
        if (++t == NT) { t = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // The whole warp runs this loop with identical values and one elected lane issues: a loop that
    // only lane 0 executes keeps descriptors in per-thread registers and costs ~70 cycles per MMA
    // in operand moves, more than a 128 x 64 x 16 MMA takes to execute.
    uint32_t it = 0, tile_it = 0;
    int t = 0, a = 0;
    uint32_t ph = 0, pha = 0;
    bool ok = true;
    WtCursor cur;
    cur.init(blockIdx.x, gridDim.x, nks, num_tiles, p.tail_split);
    WtItem w;
    for (; ok && cur.next(&w); ++tile_it) {
      if (!mbar_wait(bar_acc_empty, (tile_it & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
      tcgen05_fence_after();
      for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
        if (!mbar_wait(bar_full_tma(t), ph, abort_flag, 3)) { ok = false; break; }
        if (!mbar_wait(bar_a_full(a), pha, abort_flag, 4)) { ok = false; break; }
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < kWtBK / 16; ++kk) {
          const uint64_t db = make_sw128_desc(x_addr(t) + kk * 32);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t a_tmem = tmem_base + static_cast<uint32_t>(Cfg::kABase + (a * 2 + h) * 32 + kk * 8);
            tcgen05_mma_f16_ts_warp(tmem_base + h * MT, a_tmem, db, kIdesc, (ks != w.ks0 || kk != 0) ? 1u : 0u);
          }
        }
        tcgen05_commit_warp(bar_empty_tma(t));   // activations of this stage consumed
        tcgen05_commit_warp(bar_a_empty(a));     // A slots reusable
        if (++t == NT) { t = 0; ph ^= 1u; }
        if (++a == NA) { a = 0; pha ^= 1u; }
      }
      if (ok) tcgen05_commit_warp(bar_acc_full);
    }
    __syncwarp();
  } else {
    // ---------------------- dequantise, then drain accumulators ---------------
    constexpr int G = Cfg::kGroups, GW = Cfg::kGroupWarps;     // GW = 4 (G = 4) or 8 (G = 2)
    const int id = tid - 64;                  // 0..511
    const int dq_warp = id >> 5;              // 0..15
    const int lane_q = warp & 3;              // TMEM lane quarter this warp may touch
    const int grp_id = dq_warp / GW;          // which group of warps
    const int sub = (dq_warp % GW) >> 2;      // GW == 8: the warp's 128-column half; GW == 4: 0 (it does both)
    constexpr int NH = (GW == 4) ? 2 : 1;     // halves per warp
    const int row = lane_q * 32 + lane;       // TMEM lane = column within a half
    const uint32_t lane_addr = static_cast<uint32_t>(lane_q * 32) << 16;
    // epilogue roles (all 16 warps): which half and which part of the m range
    const int e_h = (dq_warp >> 2) & 1;
    const int e_part = dq_warp >> 3;
    const int zcols = p.N >> 3;
    uint32_t it = 0, tile_it = 0;
    // After a failed wait a warp stops computing and only walks through its remaining items.
    bool ok = true;
    int tail_seen = 0;                        // tail items this CTA has finished (it has at most two)
    WtCursor cur;
    cur.init(blockIdx.x, gridDim.x, nks, num_tiles, p.tail_split);
    WtItem w;
    for (; cur.next(&w); ++tile_it) {
      int tile_m, tile_n;
      tile_coords(w.tile, p.mtiles, p.ntiles, &tile_m, &tile_n);
      const int m0 = tile_m * MT;
      const int n0 = tile_n * kWtBN;
      int ncol[NH];
      bool nval[NH];
      uint32_t zsh[NH];
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) {
        const int h = (NH == 2) ? hh : sub;
        ncol[hh] = n0 + h * 128 + row;
        nval[hh] = ncol[hh] < p.N;
        zsh[hh] = awq_slot_shift(static_cast<uint32_t>(ncol[hh] & 7));
      }
      auto load_sz = [&](int ks, int kh, uint32_t (&s)[NH], uint32_t (&z)[NH]) {
        const int grp = (ks * kWtBK + kh * 32) / p.group_size;
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) {
          s[hh] = nval[hh] ? __ldg(p.scales + static_cast<size_t>(grp) * p.N + ncol[hh]) : 0u;
          z[hh] = nval[hh] ? __ldg(p.qzeros + static_cast<size_t>(grp) * zcols + (ncol[hh] >> 3)) : 0u;
        }
      };
      uint32_t sc[NH], zw[NH];
      uint32_t sc_hi[NH], zw_hi[NH];          // second 32 k of a stage when groups are 32 wide
      int sz_group = -1;

      for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
        if (static_cast<int>(it % G) != grp_id) continue;       // another group's stage
        const int t = it % NT, a = it % NA;
        const uint32_t ph = (it / NT) & 1u, pha = (it / NA) & 1u;
        if (!sz_by_copy) {
          const int qgrp = (ks * kWtBK) / p.group_size;
          if (half_stage_groups) { load_sz(ks, 0, sc, zw); load_sz(ks, 1, sc_hi, zw_hi); }
          else if (qgrp != sz_group) { load_sz(ks, 0, sc, zw); sz_group = qgrp; }
        }
        if (ok && !mbar_wait(bar_full_tma(t), ph, abort_flag, 5)) ok = false;
        if (!ok) continue;
        const unsigned char* raw = base_ptr + (raw_addr(t) - base);
        if (sz_by_copy) {
          const unsigned char* szp = base_ptr + (x_addr(t) - base) + Cfg::kSzOff;
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) {
            const int cl = ((NH == 2) ? hh : sub) * 128 + row;
            sc[hh] = reinterpret_cast<const uint16_t*>(szp)[cl];
            zw[hh] = reinterpret_cast<const uint32_t*>(szp + 512)[cl >> 3];
          }
        }
        uint4 r[NH][2];
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) {
          const int h = (NH == 2) ? hh : sub;
#pragma unroll
          for (int kh = 0; kh < 2; ++kh)
            r[hh][kh] = *reinterpret_cast<const uint4*>(raw + (h * 128 + row) * 32 + ((kh ^ ((row >> 2) & 1)) << 4));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty_tma(t));            // packed weights are in registers
        if (!mbar_wait(bar_a_empty(a), pha ^ 1u, abort_flag, 7)) { ok = false; continue; }
        tcgen05_fence_after();
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) {
          const int h = (NH == 2) ? hh : sub;
          ZeroPair zp = make_zero_pair((zw[hh] >> zsh[hh]) & 0xFu);
          uint32_t s2 = sc[hh] * 0x00010001u;
#pragma unroll
          for (int kh = 0; kh < 2; ++kh) {
            if (half_stage_groups && kh == 1) {                  // warp-uniform
              zp = make_zero_pair((zw_hi[hh] >> zsh[hh]) & 0xFu);
              s2 = sc_hi[hh] * 0x00010001u;
            }
            const uint32_t w[4] = {r[hh][kh].x, r[hh][kh].y, r[hh][kh].z, r[hh][kh].w};
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t q4[4];
              dequant_word(w[i], zp, s2, q4);
              o[4 * i + 0] = q4[0]; o[4 * i + 1] = q4[1]; o[4 * i + 2] = q4[2]; o[4 * i + 3] = q4[3];
            }
            tcgen05_st_32x32b_x16(tmem_base + lane_addr + static_cast<uint32_t>(Cfg::kABase + (a * 2 + h) * 32 + kh * 16), o);
          }
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_a_full(a));
      }

      // ------------------------------ epilogue --------------------------------
      // A tile of the tail that several CTAs share: contributors are the CTAs that own its first and
      // last unit and all between; this CTA's partial tile goes to its slot 2*b + (items finished).
      int nc = 1, c_first = 0;
      if (w.tail >= 0) {
        const long long t0u = static_cast<long long>(w.tail) * nks;
        c_first = stream_cta_of(t0u, cur.Ut, cur.G);
        nc = stream_cta_of(t0u + nks - 1, cur.Ut, cur.G) - c_first + 1;
      }
      const bool direct = (nc == 1);
      float* my_partial = direct ? nullptr
                                 : p.partial + static_cast<size_t>(2 * blockIdx.x + tail_seen) * (MT * kWtBN);
      if (ok && !mbar_wait(bar_acc_full, tile_it & 1u, abort_flag, 6)) ok = false;
      const int n = n0 + e_h * 128 + row;
      const bool nvalid = n < p.N;
      const uint16_t bias_n = (p.epi.bias != nullptr && nvalid) ? p.epi.bias[n] : static_cast<uint16_t>(0);
      if (ok) {
        tcgen05_fence_after();
        constexpr int kChunks = MT / 16;                 // 16 activation rows per chunk
        constexpr int kHalfChunks = (kChunks + 1) / 2;   // the two warps of a (quarter, half) split the rows
#pragma unroll 1
        for (int ch = e_part * kHalfChunks; ch < min(kChunks, (e_part + 1) * kHalfChunks); ++ch) {
          uint32_t v[16];
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
              "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
              : "r"(tmem_base + lane_addr + static_cast<uint32_t>(e_h * MT + ch * 16))
              : "memory");
          tcgen05_wait_ld();
          if (direct) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + ch * 16 + j;
              if (m < p.M) {                            // warp-uniform
                __half hv = __float2half_rn(__uint_as_float(v[j]));
                if (p.epi.bias != nullptr) hv = __hadd(hv, __ushort_as_half(bias_n));
                // 32 lanes = 32 consecutive columns starting at a multiple of 32: 64 contiguous bytes of a row
                epilogue_finish_lane(p.y, p.epi, m, p.N, n, hv, nvalid);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)      // [row of the tile][column of the tile] fp32, 32 lanes = 128 contiguous bytes
              __stcg(my_partial + (ch * 16 + j) * kWtBN + e_h * 128 + row, __uint_as_float(v[j]));
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty);
      }
      if (w.tail >= 0) ++tail_seen;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, 0x100u | static_cast<unsigned>(s_abort));
}

}  // namespace awq

namespace awq {

// Second kernel of the tail split: block (tt, chunk) adds the partial tiles of tail tile tt for 16
// of its rows, in contributor order, and writes y.  256 threads = 4 rows x 64 float4 columns at a time.
template <int MT>
__global__ void __launch_bounds__(256) wtm_fixup_kernel(const WtParams p, int G, int nks, int full_rounds,
                                                         int tail_tiles) {
  const int tt = blockIdx.x;
  const long long Ut = static_cast<long long>(tail_tiles) * nks;
  const long long t0u = static_cast<long long>(tt) * nks;
  const int c_first = stream_cta_of(t0u, Ut, G);
  const int nc = stream_cta_of(t0u + nks - 1, Ut, G) - c_first + 1;
  if (nc == 1) return;                       // finished by one CTA, which wrote y itself
  int tile_m, tile_n;
  tile_coords(full_rounds * G + tt, p.mtiles, p.ntiles, &tile_m, &tile_n);
  const int m0 = tile_m * MT, n0 = tile_n * kWtBN;
  const int col = (threadIdx.x & 63) * 4;
  const int n = n0 + col;
  const int r0 = blockIdx.y * 16 + (threadIdx.x >> 6);
  float4 sum[4];
  for (int c = 0; c < nc; ++c) {
    const int cc = c_first + c;
    const int first_tail = static_cast<int>((cc * Ut / G) / nks);
    const float* src = p.partial + static_cast<size_t>(2 * cc + (first_tail == tt ? 0 : 1)) * (MT * kWtBN) + col;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldcg(reinterpret_cast<const float4*>(src + (r0 + 4 * i) * kWtBN));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (c == 0) sum[i] = v[i];
      else { sum[i].x += v[i].x; sum[i].y += v[i].y; sum[i].z += v[i].z; sum[i].w += v[i].w; }
    }
  }
  if (n >= p.N) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + r0 + 4 * i;
    if (m >= p.M) continue;
    __half2 lo = __floats2half2_rn(sum[i].x, sum[i].y), hi = __floats2half2_rn(sum[i].z, sum[i].w);
    if (p.epi.bias != nullptr) {
      lo = __hadd2(lo, *reinterpret_cast<const __half2*>(p.epi.bias + n));
      hi = __hadd2(hi, *reinterpret_cast<const __half2*>(p.epi.bias + n + 2));
    }
    const uint32_t words[2] = {*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi)};
    epilogue_finish_words<2>(p.y, p.epi, m, p.N, n, words);
  }
}

}  // namespace awq

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
namespace awq {

// Workspace layout of the GEMM entry points: [0, 256) status word; [256, 256 + 16 KiB) left alone (the
// decode kernels keep their arrival counters there when awq_b200_linear shares the buffer); then the
// fp32 partial tiles of the tail split, which need no initialisation.
constexpr size_t kWtPartialOff = 256 + 16384;

size_t wtm_workspace_bytes(int sm_count) {
  return kWtPartialOff + static_cast<size_t>(sm_count) * 2 * 192 * kWtBN * sizeof(float);
}

template <int MT>
static int launch_wtm(const void* x, const void* packed, WtParams p, int sm_count, EncodeTiledFn encode,
                      cudaStream_t stream, size_t workspace_bytes) {
  using Cfg = WtCfg<MT>;
  CUtensorMap mx, mw;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.K) * 2};
    const cuuint32_t box[2] = {kWtBK, MT};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.K / kBlockK)};
    const cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(p.N) * 64};
    const cuuint32_t box[3] = {32, kWtBN, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(packed), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  p.mtiles = (p.M + MT - 1) / MT;
  p.ntiles = (p.N + kWtBN - 1) / kWtBN;
  AWQ_CUDA_TRY(cudaFuncSetAttribute(wtm_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  const int tiles = p.mtiles * p.ntiles;
  // Tail split: worth it when the last wave is partial - or the only wave leaves SMs idle - and the idle
  // time it would leave (a fraction of one tile's k loop) clearly exceeds the cost of the partial tiles
  // (~10 us), and the caller's workspace has room for two fp32 tiles per CTA.  With fewer tiles than SMs
  // every tile is then cut along k and all SMs work (full_rounds = 0).
  const int tail = tiles % sm_count;   // with fewer tiles than SMs: all of them
  const double idle_us = tail ? (1.0 - static_cast<double>(tail) / sm_count) * (p.K / kWtBK) * 0.6 : 0.0;
  const size_t need = kWtPartialOff + static_cast<size_t>(sm_count) * 2 * MT * kWtBN * sizeof(float);
  p.tail_split = (idle_us > 35.0 && p.partial != nullptr && workspace_bytes >= need) ? 1 : 0;
  // Every CTA of a split grid must own at least one unit (the fix-up adds the slots of all CTAs between a
  // tile's first and last contributor): no more CTAs than units.
  const long long units = static_cast<long long>(tiles) * (p.K / kWtBK);
  const int grid = p.tail_split ? static_cast<int>(units < sm_count ? units : sm_count)
                                : (tiles < sm_count ? tiles : sm_count);
  wtm_kernel<MT><<<grid, kWtThreads, Cfg::kSmemBytes, stream>>>(mx, mw, p);
  AWQ_CUDA_TRY(cudaGetLastError());
  if (p.tail_split) {
    const int full_rounds = tiles / grid;   // 0 when every tile is split
    wtm_fixup_kernel<MT><<<dim3(tail, MT / 16), 256, 0, stream>>>(p, grid, p.K / kWtBK, full_rounds, tail);
    AWQ_CUDA_TRY(cudaGetLastError());
  }
  return AWQ_B200_OK;
}

int wtm_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                 void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream, int m_tile) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size, true)) return st;
  if (M < 1) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) || !aligned16(y))
    return AWQ_B200_ERR_ALIGN;
  if (int st = check_epilogue(epi, N)) return st;
  if (!workspace || workspace_bytes < 16) return AWQ_B200_ERR_WORKSPACE;
  if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;
  EncodeTiledFn encode;
  if (int st = get_encode(&encode)) return st;
  WtParams p;
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.epi = epi;
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  const bool roomy = workspace_bytes > kWtPartialOff;
  p.partial = roomy ? reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kWtPartialOff) : nullptr;
  p.M = M; p.K = K; p.N = N;
  p.group_size = group_size;
  p.mtiles = p.ntiles = 0;
  p.tail_split = 0;
  if (m_tile == 0) m_tile = M <= 64 ? 64 : (M <= 128 ? 128 : 192);
  switch (m_tile) {
    case 64: return launch_wtm<64>(x, packed, p, di.sm_count, encode, stream, workspace_bytes);
    case 128: return launch_wtm<128>(x, packed, p, di.sm_count, encode, stream, workspace_bytes);
    case 192: return launch_wtm<192>(x, packed, p, di.sm_count, encode, stream, workspace_bytes);
    default: return AWQ_B200_ERR_SHAPE;
  }
}

}  // namespace awq

extern "C" {

// Same contract as awq_b200_gemm (workspace = one zero-initialised status word); the weights take the
// tensor-memory route.  Kept as a separate entry point so that the two GEMM kernels can be compared.
int awq_b200_gemm_wtm(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                      void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                      awq_b200_stream_t stream) {
  return awq::wtm_dispatch(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream), 0);
}

// Tuning hook: the same with the activation-row tile forced (64, 128 or 192; 0 = by M).
int awq_b200_gemm_wtm_tile(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                           const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                           size_t workspace_bytes, awq_b200_stream_t stream, int m_tile) {
  return awq::wtm_dispatch(x, packed, scales, qzeros, awq::Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream), m_tile);
}

}  // extern "C"
