// 8-bit quantized linears of the reference runtime on tcgen05: FP8 (e4m3 x e4m3 -> fp32) and SmoothQuant INT8
// (s8 x s8 -> s32), both operands K-major as the reference hands them over (activations [M, K] row-major, weights
// [N, K] row-major, i.e. the `qweight.t()` view the reference passes).
//
//   tensorwise  y = alpha * (x . w^T) + beta * bias          cutlass_f8f8bf16_tensorwise_sm89
//                                                            (LLMQRT/runtime_refact/csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:30-160)
//                                                            w8a8_int8_linear_bbf16_obf16_per_tensor
//                                                            (LLMQRT/runtime_refact/csrc/smoothquant/sq_gemm.cu:30-170)
//   rowwise     y = (x . w^T) * x_scale[m] * w_scale[n] + bias    cutlass_f8f8bf16_rowwise_sm89
//                                                            (LLMQRT/runtime_refact/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:425-2248)
//
// One persistent kernel: CTA tile = 128 or 256 weight rows (one or two tcgen05 M = 128 halves: the weights are the A
// operand, so a thread's tensor-memory lane is an output column) x MT activation rows (the MMA's N), K walked in
// stages of 128 bytes.  Warp 0 copies both operands with TMA (128-byte swizzle), warp 1 issues the MMAs (K = 32 per
// instruction), warps 2..9 drain the accumulators: two accumulator sets in tensor memory, so the epilogue of a work
// item overlaps the MMAs of the next.  No quantisation happens here: the operands arrive quantised, as in the
// reference.  Every mbarrier wait is bounded (see awq_ptx.cuh).  Up to 128 rows: tiles of 128 weight rows x
// 32 / 64 / 128 activation rows, two CTAs per SM (the weights are streamed once: bytes in flight and overlapped
// epilogues matter, not the tile's arithmetic intensity); more rows: 256 x 128 tiles, one CTA per SM.
//
// Few rows make few tiles (a decode step has N / 128 of them), so a tile's K range can be split over the CTAs of
// one thread-block cluster (2..8): each leaves its 32-bit partial sums in its own shared memory (the operand ring
// is free by then), and after a cluster barrier every CTA adds, IN SPLIT ORDER, the partials of its share of the
// tile's rows out of all the peers' shared memory and writes those rows.  The order is fixed, so fp8 results
// are the same on every call; int32 partials are exact in any order.  No workspace, no atomics.
#include <cuda_bf16.h>

#include "awq_common.cuh"
#include "awq_gemv_common.cuh"
#include "awq_ptx.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kQ8Threads = 64 + 256;         // producer, issuer, 8 epilogue warps
constexpr int kQ8BK = 128;                   // bytes of K per stage
constexpr int kQ8MaxSplits = 8;              // portable cluster size

// MT activation rows and HALVES x 128 weight rows per tile.
template <int MT, int HALVES> struct Q8Cfg {
  static_assert(MT == 32 || MT == 64 || MT == 128, "activation rows per tile");
  static_assert(HALVES == 1 || HALVES == 2, "weight rows per tile: 128 or 256");
  static constexpr int kBN = 128 * HALVES;
  static constexpr int kABytes = kBN * kQ8BK;
  static constexpr int kBBytes = MT * kQ8BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // 128-wide tiles: two CTAs per SM (one drains / reduces while the other streams); 256-wide tiles: one
  static constexpr int kCtasPerSm = HALVES == 1 ? 2 : 1;
  static constexpr int kBudget = kCtasPerSm == 2 ? 104 * 1024 : 200 * 1024;
  static constexpr int kStages = kBudget / kStageBytes >= 6 ? 6 : kBudget / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kAccCols = HALVES * MT;                  // one accumulator set
  static constexpr int kTmemCols = 2 * kAccCols <= 32 ? 32 : (2 * kAccCols <= 64 ? 64 : (2 * kAccCols <= 128 ? 128 : (2 * kAccCols <= 256 ? 256 : 512)));
};

struct Q8Params {
  void* y;                 // [M, N] bf16 or fp16
  const void* bias;        // [N], or null
  const float* alpha_dev;  // tensorwise: optional device scalars multiplied into alpha (activation scale,
  const float* alpha_dev2; // weight scale), so that a dynamic scale needs no host round trip
  const float* x_scale;    // rowwise: [M]
  const float* w_scale;    // rowwise: [N]
  float alpha, beta;
  unsigned* status;
  int M, N, K;
  int mtiles, ntiles;
  int splits, kper;        // K split: work item = (tile, split), split s walks stages [s * kper, (s + 1) * kper)
  int ldx, ldw;            // row pitches of the activations and of the weights, in bytes
  int rowwise;             // 0 tensorwise, 1 rowwise
  int out_bf16;            // 1 bf16, 0 fp16
  int bias_kind;           // 0 none, 1 bf16, 2 fp16, 3 fp32
  uint32_t idesc;          // instruction descriptor (operand formats, tile shape)
};

// Instruction descriptors, both operands K-major.  kind::i8: D s32 (2 at bit 4), A and B s8 (1 at bits 7 and 10).
// kind::f8f6f4: D fp32 (1 at bit 4), A = the weights e4m3 (0 at bit 7), B = the activations e4m3 (0) or e5m2 (1) at
// bit 10.
__host__ __device__ constexpr uint32_t make_q8_idesc(bool is_int, bool x_e5m2, int m, int n) {
  return (is_int ? ((2u << 4) | (1u << 7) | (1u << 10)) : ((1u << 4) | (x_e5m2 ? (1u << 10) : 0u))) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Four k steps (32 bytes each) of one 128-byte stage for one half, then optionally commits, one election.
template <bool INT8>
__device__ __forceinline__ void q8_mma_stage_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate_first) {
  if constexpr (INT8) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b32 alo, ahi, blo, bhi;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "mov.b64 {alo, ahi}, %1;\n\t  mov.b64 {blo, bhi}, %2;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b32 alo, ahi, blo, bhi;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "mov.b64 {alo, ahi}, %1;\n\t  mov.b64 {blo, bhi}, %2;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t"
        "add.u32 alo, alo, 2;\n\t  add.u32 blo, blo, 2;\n\t  mov.b64 da, {alo, ahi};\n\t  mov.b64 db, {blo, bhi};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first)
        : "memory");
  }
}

// CLUSTER: one work item per CTA, the p.splits CTAs of a cluster share a tile (cluster rank = split).
template <bool INT8, int MT, int HALVES, bool CLUSTER>
__global__ void __launch_bounds__(kQ8Threads, Q8Cfg<MT, HALVES>::kCtasPerSm)
q8_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Q8Params p) {
  using Cfg = Q8Cfg<MT, HALVES>;
  constexpr int NT = Cfg::kStages;
  constexpr int BN = Cfg::kBN;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem_base;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto a_addr = [&](int t) { return base + t * Cfg::kStageBytes; };
  auto b_addr = [&](int t) { return base + t * Cfg::kStageBytes + Cfg::kABytes; };
  const uint32_t bar_base = base + NT * Cfg::kStageBytes;
  auto bar_full = [&](int t) { return bar_base + 8u * t; };
  auto bar_empty = [&](int t) { return bar_base + 8u * (NT + t); };
  auto bar_acc_full = [&](int s) { return bar_base + 8u * (2 * NT + s); };
  auto bar_acc_empty = [&](int s) { return bar_base + 8u * (2 * NT + 2 + s); };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_full(t), 1);
      mbar_init(bar_empty(t), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_acc_full(s), 1);
      mbar_init(bar_acc_empty(s), 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  const int nks = (p.K + kQ8BK - 1) / kQ8BK;          // the copy zero-fills the last stage beyond K
  const int num_items = p.mtiles * p.ntiles * p.splits;
  const uint32_t kIdesc = p.idesc;
  // work item -> (column tile, row tile, split); the splits of a tile are neighbours, so they run at the same time
  auto decode = [&](int item, int* tn, int* tm, int* k0, int* k1) {
    const int tile = item / p.splits, split = item - tile * p.splits;
    *tn = tile / p.mtiles;
    *tm = tile - *tn * p.mtiles;           // row tiles fastest: a wave shares weight tiles
    *k0 = split * p.kper;
    *k1 = min(nks, *k0 + p.kper);
  };

  if (warp == 0) {
    // ------------------------------ copy producer ------------------------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      int tn, tm, k0, k1;
      decode(item, &tn, &tm, &k0, &k1);
      for (int ks = k0; ks < k1; ++ks, ++it) {
        const int t = it % NT;
        if (it >= static_cast<uint32_t>(NT) &&
            !mbar_wait(bar_empty(t), ((it / NT) - 1u) & 1u, abort_flag, 1)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar_full(t), Cfg::kStageBytes);
          tma_load_2d(a_addr(t), &map_w, ks * kQ8BK, tn * BN, bar_full(t));
          tma_load_2d(b_addr(t), &map_x, ks * kQ8BK, tm * MT, bar_full(t));
        }
        __syncwarp();
      }
    }
    // leave only after the last copies have landed (bounded)
    const uint32_t issued = it;
    for (uint32_t j = issued > static_cast<uint32_t>(NT) ? issued - NT : 0u; j < issued; ++j)
      mbar_wait_timed(bar_full(j % NT), (j / NT) & 1u);
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    uint32_t it = 0, item_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++item_it) {
      int tn, tm, k0, k1;
      decode(item, &tn, &tm, &k0, &k1);
      const uint32_t set = item_it & 1u;
      if (!mbar_wait(bar_acc_empty(set), ((item_it >> 1) & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + set * Cfg::kAccCols;
      for (int ks = k0; ks < k1; ++ks, ++it) {
        const int t = it % NT;
        if (!mbar_wait(bar_full(t), (it / NT) & 1u, abort_flag, 3)) { ok = false; break; }
        tcgen05_fence_after();
        const uint64_t bd = make_sw128_desc(b_addr(t));
        q8_mma_stage_warp<INT8>(acc, make_sw128_desc(a_addr(t)), bd, kIdesc, ks != k0 ? 1u : 0u);
        if constexpr (HALVES == 2)
          q8_mma_stage_warp<INT8>(acc + MT, make_sw128_desc(a_addr(t) + 128 * kQ8BK), bd, kIdesc, ks != k0 ? 1u : 0u);
        tcgen05_commit_warp(bar_empty(t));
      }
      if (ok) tcgen05_commit_warp(bar_acc_full(set));
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------------
    // Warp (quarter q, part h): lanes = output columns n0 + 32q + lane of half h (HALVES == 2: warps 2..5 take half 0,
    // 6..9 half 1; HALVES == 1: the two warps of a quarter share the accumulator's columns, i.e. the rows of x).
    const int ew = warp - 2;                 // 0..7
    const int lane_q = warp & 3;
    const int part = ew >> 2;                // 0 or 1
    const int h = HALVES == 2 ? part : 0;
    constexpr int kRowStep = HALVES == 2 ? 32 : 64;          // rows of x between this warp's 32-row loads
    const int row_first = HALVES == 2 ? 0 : part * 32;
    const uint32_t lane_addr = static_cast<uint32_t>(lane_q * 32) << 16;
    const int col = h * 128 + lane_q * 32 + lane;            // column inside the tile
    uint32_t item_it = 0;
    bool ok = true;
    float alpha = p.alpha;
    if (!p.rowwise && p.alpha_dev != nullptr) alpha = __fmul_rn(alpha, __ldg(p.alpha_dev));
    if (!p.rowwise && p.alpha_dev2 != nullptr) alpha = __fmul_rn(alpha, __ldg(p.alpha_dev2));

    auto finish = [&](uint32_t raw, int m, int n, float ws_n, float bias_n, float beta_bias) {
      const float a = INT8 ? static_cast<float>(static_cast<int>(raw)) : __uint_as_float(raw);
      float r;
      if (p.rowwise) r = __fadd_rn(__fmul_rn(__fmul_rn(a, __ldg(p.x_scale + m)), ws_n), bias_n);
      else r = fmaf(alpha, a, beta_bias);
      const size_t at = static_cast<size_t>(m) * p.N + n;
      if (p.out_bf16) static_cast<__nv_bfloat16*>(p.y)[at] = __float2bfloat16_rn(r);
      else static_cast<__half*>(p.y)[at] = __float2half_rn(r);
    };

    for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++item_it) {
      int tn, tm, k0, k1;
      decode(item, &tn, &tm, &k0, &k1);
      const uint32_t set = item_it & 1u;
      const int n = tn * BN + col;
      const bool nvalid = n < p.N;
      float bias_n = 0.f, ws_n = 1.f;
      if (nvalid) {
        if (p.bias_kind == 1) bias_n = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
        else if (p.bias_kind == 2) bias_n = __half2float(static_cast<const __half*>(p.bias)[n]);
        else if (p.bias_kind == 3) bias_n = static_cast<const float*>(p.bias)[n];
        if (p.rowwise) ws_n = __ldg(p.w_scale + n);
      }
      const float beta_bias = __fmul_rn(p.beta, bias_n);
      if (ok && !mbar_wait(bar_acc_full(set), (item_it >> 1) & 1u, abort_flag, 4)) ok = false;
      if (ok) {
        tcgen05_fence_after();
#pragma unroll 1
        for (int c0 = row_first; c0 < MT; c0 += kRowStep) {
          if (tm * MT + c0 >= p.M) break;                       // rows beyond M are padding (warp-uniform)
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_base + lane_addr + set * Cfg::kAccCols + h * MT + c0, v);
          tcgen05_wait_ld();
          if constexpr (!CLUSTER) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int m = tm * MT + c0 + j;
              if (m < p.M && nvalid) finish(v[j], m, n, ws_n, bias_n, beta_bias);
            }
          } else {
            // partial sums of this split: [row][column] words at the start of the (now idle) operand ring
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (tm * MT + c0 + j < p.M)
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + 4u * ((c0 + j) * BN + col)), "r"(v[j]) : "memory");
          }
        }
        tcgen05_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(set));
    }
  }

  if constexpr (CLUSTER) {
    // Every thread of every CTA of the cluster: partials are in place.
    cluster_sync_all();
    if (warp >= 2) {
      int tn, tm, k0, k1;
      decode(blockIdx.x, &tn, &tm, &k0, &k1);
      const int rank = blockIdx.x % p.splits;
      const int et = tid - 64;                                   // 0..255
      const int col = et % BN;
      const int rows_valid = min(MT, p.M - tm * MT);
      const int n = tn * BN + col;
      if (n < p.N) {
        float bias_n = 0.f, ws_n = 1.f;
        if (p.bias_kind == 1) bias_n = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
        else if (p.bias_kind == 2) bias_n = __half2float(static_cast<const __half*>(p.bias)[n]);
        else if (p.bias_kind == 3) bias_n = static_cast<const float*>(p.bias)[n];
        if (p.rowwise) ws_n = __ldg(p.w_scale + n);
        const float beta_bias = __fmul_rn(p.beta, bias_n);
        float alpha = p.alpha;
        if (!p.rowwise && p.alpha_dev != nullptr) alpha = __fmul_rn(alpha, __ldg(p.alpha_dev));
        if (!p.rowwise && p.alpha_dev2 != nullptr) alpha = __fmul_rn(alpha, __ldg(p.alpha_dev2));
        // this CTA's share: rows rank, rank + splits, ... ; the thread walks them 256 / BN apart
        for (int row = rank + (et / BN) * p.splits; row < rows_valid; row += (256 / BN) * p.splits) {
          const uint32_t local = base + 4u * (row * BN + col);
          uint32_t part[kQ8MaxSplits];
#pragma unroll
          for (int sp = 0; sp < kQ8MaxSplits; ++sp) {
            if (sp < p.splits) {
              uint32_t remote;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(sp));
              asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(part[sp]) : "r"(remote) : "memory");
            }
          }
          float a;
          if constexpr (INT8) {
            int acc = 0;
#pragma unroll
            for (int sp = 0; sp < kQ8MaxSplits; ++sp)
              if (sp < p.splits) acc += static_cast<int>(part[sp]);
            a = static_cast<float>(acc);
          } else {
            a = __uint_as_float(part[0]);
#pragma unroll
            for (int sp = 1; sp < kQ8MaxSplits; ++sp)
              if (sp < p.splits) a = __fadd_rn(a, __uint_as_float(part[sp]));
          }
          const int m = tm * MT + row;
          float r;
          if (p.rowwise) r = __fadd_rn(__fmul_rn(__fmul_rn(a, __ldg(p.x_scale + m)), ws_n), bias_n);
          else r = fmaf(alpha, a, beta_bias);
          const size_t at = static_cast<size_t>(m) * p.N + n;
          if (p.out_bf16) static_cast<__nv_bfloat16*>(p.y)[at] = __float2bfloat16_rn(r);
          else static_cast<__half*>(p.y)[at] = __float2half_rn(r);
        }
      }
    }
    cluster_sync_all();                                          // nobody leaves while its shared memory may be read
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, 0x500u | static_cast<unsigned>(s_abort));
}

// How a problem is cut: tile shape by row count, then a K split when the tiles alone would leave SMs idle.
struct Q8Plan {
  int mt, halves, mtiles, ntiles, splits, kper;
};
static Q8Plan q8_plan(int M, int N, int K, int sm_count, bool allow_split) {
  Q8Plan pl{};
  // up to 128 rows: many small CTAs (128 weight rows each), two per SM; beyond that the tile is 256 x 128
  pl.mt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  pl.halves = M <= 128 ? 1 : 2;
  const int bn = 128 * pl.halves;
  const int ctas = (pl.halves == 1 ? 2 : 1) * sm_count;
  pl.mtiles = (M + pl.mt - 1) / pl.mt;
  pl.ntiles = (N + bn - 1) / bn;
  const int tiles = pl.mtiles * pl.ntiles;
  const int nks = (K + kQ8BK - 1) / kQ8BK;
  int splits = 1;
  if (allow_split && tiles * 4 < ctas * 3) {
    splits = ctas / tiles;                                   // all work items resident at once
    const int max_by_k = nks / 4 > 1 ? nks / 4 : 1;          // at least four stages per split
    if (splits > max_by_k) splits = max_by_k;
    if (splits > kQ8MaxSplits) splits = kQ8MaxSplits;
  }
  pl.kper = (nks + splits - 1) / splits;
  pl.splits = (nks + pl.kper - 1) / pl.kper;                 // no empty split
  return pl;
}

template <bool INT8, int MT, int HALVES>
static int launch_q8(const void* x, const void* w, Q8Params p, const Q8Plan& pl, int sm_count, EncodeTiledFn encode,
                     cudaStream_t stream) {
  using Cfg = Q8Cfg<MT, HALVES>;
  CUtensorMap mx, mw;
  const cuuint32_t estr[2] = {1, 1};
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldx)};
    const cuuint32_t box[2] = {kQ8BK, MT};
    if (encode(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(x), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cuda_fail(cudaErrorInvalidValue);
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.N)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldw)};
    const cuuint32_t box[2] = {kQ8BK, static_cast<cuuint32_t>(Cfg::kBN)};
    if (encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cuda_fail(cudaErrorInvalidValue);
  }
  p.idesc = make_q8_idesc(INT8, p.idesc != 0u, 128, MT);
  p.mtiles = pl.mtiles;
  p.ntiles = pl.ntiles;
  p.splits = pl.splits;
  p.kper = pl.kper;
  const int items = pl.mtiles * pl.ntiles * pl.splits;
  const int resident = Cfg::kCtasPerSm * sm_count;
  if (pl.splits > 1) {
    // one work item per CTA; the splits of a tile are the CTAs of one cluster
    auto kernel = q8_gemm_kernel<INT8, MT, HALVES, true>;
    AWQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    AWQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(items);
    cfg.blockDim = dim3(kQ8Threads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(pl.splits);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, mx, mw, p));
    return AWQ_B200_OK;
  }
  auto kernel = q8_gemm_kernel<INT8, MT, HALVES, false>;
  AWQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  AWQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  kernel<<<items < resident ? items : resident, kQ8Threads, Cfg::kSmemBytes, stream>>>(mx, mw, p);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

static int q8_dispatch(bool is_int, const void* x, const void* w, Q8Params p, unsigned flags, cudaStream_t stream) {
  if (!x || !w || !p.y) return AWQ_B200_ERR_NULL;
  if (p.M < 1 || p.N < 1 || p.K < 1) return AWQ_B200_ERR_SHAPE;
  // the bulk tensor copies want row pitches that are multiples of 16 bytes
  if (p.ldx < p.K || p.ldw < p.K || (p.ldx % 16) != 0 || (p.ldw % 16) != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(w) || (reinterpret_cast<uintptr_t>(p.y) & 1u)) return AWQ_B200_ERR_ALIGN;
  if (p.rowwise && (!p.x_scale || !p.w_scale)) return AWQ_B200_ERR_NULL;
  if (p.bias_kind < 0 || p.bias_kind > 3 || ((p.bias_kind != 0) != (p.bias != nullptr))) return AWQ_B200_ERR_SHAPE;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;
  EncodeTiledFn encode;
  if (int st = get_encode(&encode)) return st;
  const Q8Plan pl = q8_plan(p.M, p.N, p.K, di.sm_count, (flags & AWQ_B200_Q8_NO_SPLIT) == 0);
  if (is_int) {
    if (pl.mt == 32) return launch_q8<true, 32, 1>(x, w, p, pl, di.sm_count, encode, stream);
    if (pl.mt == 64) return launch_q8<true, 64, 1>(x, w, p, pl, di.sm_count, encode, stream);
    if (pl.halves == 1) return launch_q8<true, 128, 1>(x, w, p, pl, di.sm_count, encode, stream);
    return launch_q8<true, 128, 2>(x, w, p, pl, di.sm_count, encode, stream);
  }
  if (pl.mt == 32) return launch_q8<false, 32, 1>(x, w, p, pl, di.sm_count, encode, stream);
  if (pl.mt == 64) return launch_q8<false, 64, 1>(x, w, p, pl, di.sm_count, encode, stream);
  if (pl.halves == 1) return launch_q8<false, 128, 1>(x, w, p, pl, di.sm_count, encode, stream);
  return launch_q8<false, 128, 2>(x, w, p, pl, di.sm_count, encode, stream);
}

}  // namespace awq

extern "C" {

int awq_b200_q8_splits(int M, int N, int K) {
  awq::DeviceInfo di;
  if (M < 1 || N < 1 || K < 1 || awq::device_info(&di)) return 0;
  return awq::q8_plan(M, N, K, di.sm_count, true).splits;
}

int awq_b200_fp8_gemm_tensorwise(const void* xq, int ldx, const void* wq, int ldw, const void* bias, int bias_kind,
                                 void* y, int M, int N, int K, float alpha, const float* alpha_dev,
                                 const float* alpha_dev2, float beta, int out_bf16, unsigned flags, unsigned* status,
                                 awq_b200_stream_t stream) {
  awq::Q8Params p{};
  p.y = y; p.bias = bias; p.bias_kind = bias_kind; p.alpha_dev = alpha_dev; p.alpha_dev2 = alpha_dev2; p.alpha = alpha;
  p.beta = beta; p.status = status; p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldw = ldw; p.rowwise = 0;
  p.out_bf16 = out_bf16; p.idesc = 0u;
  return awq::q8_dispatch(false, xq, wq, p, flags, static_cast<cudaStream_t>(stream));
}

int awq_b200_fp8_gemm_rowwise(const void* xq, int ldx, int x_is_e5m2, const void* wq, int ldw, const void* bias,
                              int bias_kind, const float* x_scale, const float* w_scale, void* y, int M, int N, int K,
                              unsigned flags, unsigned* status, awq_b200_stream_t stream) {
  awq::Q8Params p{};
  p.y = y; p.bias = bias; p.bias_kind = bias_kind; p.x_scale = x_scale; p.w_scale = w_scale; p.alpha = 1.f;
  p.beta = 1.f; p.status = status; p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldw = ldw; p.rowwise = 1; p.out_bf16 = 1;
  p.idesc = x_is_e5m2 ? 1u : 0u;
  return awq::q8_dispatch(false, xq, wq, p, flags, static_cast<cudaStream_t>(stream));
}

int awq_b200_int8_gemm_tensorwise(const void* xq, int ldx, const void* wq, int ldw, const void* bias, int bias_kind,
                                  void* y, int M, int N, int K, float alpha, const float* alpha_dev,
                                  const float* alpha_dev2, float beta, int out_bf16, unsigned flags, unsigned* status,
                                  awq_b200_stream_t stream) {
  awq::Q8Params p{};
  p.y = y; p.bias = bias; p.bias_kind = bias_kind; p.alpha_dev = alpha_dev; p.alpha_dev2 = alpha_dev2; p.alpha = alpha;
  p.beta = beta; p.status = status; p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldw = ldw; p.rowwise = 0;
  p.out_bf16 = out_bf16; p.idesc = 0u;
  return awq::q8_dispatch(true, xq, wq, p, flags, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
