// Prefill path: W4A16 GEMM on 5th-generation tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM, CTA tile (128*MH) x 256,
// k-stage of 64:
//   warp 0      TMA producer: activations [128 x 64] fp16 per row half (128-byte
//               swizzle) and the packed int4 weights [256 columns x 32 bytes].
//   warp 1      allocates tensor memory and issues tcgen05.mma (M=128, N=256,
//               K=16, fp16 inputs, fp32 accumulators in TMEM), one thread.
//   warps 2-17  read the packed nibbles from shared memory, dequantise them to
//               the exact reference fp16 weight and store them as the K-major,
//               128-byte-swizzled B operand; after the last k-stage the same
//               warps drain the accumulators (tcgen05.ld), round to fp16, add
//               the bias and store Y.
// Stages are handed over with mbarriers.  Every wait is bounded: on expiry the
// kernel raises an abort flag, all roles fall through, tensor memory is freed
// and a non-zero status word is left in the workspace.
#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int kDequantThreads = 512;              // 16 warps: dequantise, then drain the accumulators
constexpr int kGemmThreads = 64 + kDequantThreads;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kABytesHalf = 128 * kBK * 2;   // 16 KiB: 128 rows x 128 B
constexpr int kBBytes = kBN * kBK * 2;       // 32 KiB: 256 columns x 128 B
constexpr int kRawBytes = kBN * (kBK / 2);   // 8 KiB: 256 columns x 32 B of nibbles

template <int MH> struct GemmCfg {
  // Two rings.  The TMA ring (activations + packed weights) is deep enough to cover the copy
  // latency; the B ring (dequantised operand) only has to let the dequantisation of stage s+1
  // overlap the MMAs of stage s.
  static constexpr int kTmaStages = (MH == 2) ? 4 : 5;
  static constexpr int kBStages = (MH == 2) ? 2 : 3;
  static constexpr int kTmaStageBytes = MH * kABytesHalf + kRawBytes;
  static constexpr int kTmemCols = 256 * MH;
  static constexpr int kSmemBytes = kTmaStages * kTmaStageBytes + kBStages * kBBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmParams {
  const uint16_t* scales;
  const uint32_t* qzeros;
  Epilogue epi;
  uint16_t* y;
  unsigned* status;  // workspace word: 0 = ok, else which wait expired
  int M, K, N;
  int group_size;
  int mtiles, ntiles;
};

// Instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) |
                                (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);

__device__ __forceinline__ uint32_t cvt_pack_bias(float a, float b, uint32_t bias2, bool has_bias) {
  __half2 h = __floats2half2_rn(a, b);
  uint32_t v = *reinterpret_cast<uint32_t*>(&h);
  if (has_bias) asm("add.f16x2 %0, %1, %2;" : "=r"(v) : "r"(v), "r"(bias2));
  return v;
}

template <int MH>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
            const GemmParams p) {
  using Cfg = GemmCfg<MH>;
  constexpr int NT = Cfg::kTmaStages, NB = Cfg::kBStages;
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem_base;

  // 1024-byte aligned carve-up: [B operand] x NB, [A halves | raw] x NT, then barriers.
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t tma_base = base + NB * kBBytes;
  auto b_addr = [&](int b) { return base + b * kBBytes; };
  auto a_addr = [&](int t, int h) { return tma_base + t * Cfg::kTmaStageBytes + h * kABytesHalf; };
  auto raw_addr = [&](int t) { return tma_base + t * Cfg::kTmaStageBytes + MH * kABytesHalf; };
  const uint32_t bar_base = tma_base + NT * Cfg::kTmaStageBytes;
  auto bar_full_tma = [&](int t) { return bar_base + 8u * t; };
  auto bar_empty_tma = [&](int t) { return bar_base + 8u * (NT + t); };   // MMA commit + 8 dequant warps
  auto bar_full_b = [&](int b) { return bar_base + 8u * (2 * NT + b); };
  auto bar_empty_b = [&](int b) { return bar_base + 8u * (2 * NT + NB + b); };
  const uint32_t bar_acc_full = bar_base + 8u * (2 * NT + 2 * NB);
  const uint32_t bar_acc_empty = bar_base + 8u * (2 * NT + 2 * NB + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    s_abort = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_full_tma(t), 1);
      mbar_init(bar_empty_tma(t), 1 + kDequantThreads / 32);
    }
    for (int b = 0; b < NB; ++b) {
      mbar_init(bar_full_b(b), kDequantThreads / 32);
      mbar_init(bar_empty_b(b), 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, kDequantThreads / 32);
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

  const int nks = p.K / kBK;
  const int num_tiles = p.mtiles * p.ntiles;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // Warp-uniform loop; lanes 0..MH-1 issue the activation boxes, lane MH the packed weights.
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    uint32_t it = 0;
    int st = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tile_m, tile_n;
      tile_coords(tile, p.mtiles, p.ntiles, &tile_m, &tile_n);
      const int m0 = tile_m * (128 * MH);
      const int n0 = tile_n * kBN;
      for (int ks = 0; ks < nks; ++ks, ++it) {
        if (!mbar_wait(bar_empty_tma(st), ph ^ 1u, abort_flag, 1)) { ok = false; break; }
        const uint32_t bar = bar_full_tma(st);
        if (lane == 0) mbar_expect_tx(bar, MH * kABytesHalf + kRawBytes);
        if (lane < MH) tma_load_2d(a_addr(st, lane), &map_x, ks * kBK, m0 + lane * 128, bar);
        if (lane == MH) tma_load_3d(raw_addr(st), &map_w, (ks & 1) * 32, n0, ks >> 1, bar);
        if (++st == NT) { st = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // Warp-uniform loop, one elected lane issues (see tcgen05_mma_f16_warp).
    uint32_t it = 0, tile_it = 0;
    int st = 0, sb = 0;
    uint32_t ph = 0, phb = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_it) {
      if (!mbar_wait(bar_acc_empty, (tile_it & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
      tcgen05_fence_after();
      for (int ks = 0; ks < nks; ++ks, ++it) {
        if (!mbar_wait(bar_full_tma(st), ph, abort_flag, 3)) { ok = false; break; }
        if (!mbar_wait(bar_full_b(sb), phb, abort_flag, 4)) { ok = false; break; }
        tcgen05_fence_after();
#pragma unroll
        for (int h = 0; h < MH; ++h) {
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t da = make_sw128_desc(a_addr(st, h) + kk * 32);
            const uint64_t db = make_sw128_desc(b_addr(sb) + kk * 32);
            tcgen05_mma_f16_warp(tmem_base + h * 256, da, db, kInstrDesc, (ks | kk) != 0 ? 1u : 0u);
          }
        }
        tcgen05_commit_warp(bar_empty_tma(st));   // activations of this stage consumed
        tcgen05_commit_warp(bar_empty_b(sb));     // B buffer reusable
        if (++st == NT) { st = 0; ph ^= 1u; }
        if (++sb == NB) { sb = 0; phb ^= 1u; }
      }
      if (ok) tcgen05_commit_warp(bar_acc_full);
    }
    __syncwarp();
  } else {
    // ---------------------- dequantise, then drain accumulators ---------------
    const int id = tid - 64;                 // 0..511
    const int dq_warp = id >> 5;             // 0..15
    const int col_local = id >> 1;           // 0..255: the column this thread dequantises
    const int hh = id & 1;                   // which 16-byte half of the column's 32 raw bytes
    const int lane_q = warp & 3;             // TMEM lane quarter this warp may read
    const int col_quarter = dq_warp >> 2;    // epilogue: columns [64*col_quarter, +64)
    // B-operand byte offsets of the four 16-byte chunks this thread writes per stage
    uint32_t boff[4];
    {
      const int r8 = col_local & 7;
      const uint32_t row_off = static_cast<uint32_t>(col_local >> 3) * 1024u + static_cast<uint32_t>(r8) * 128u;
#pragma unroll
      for (int i = 0; i < 4; ++i) boff[i] = row_off + static_cast<uint32_t>(((4 * hh + i) ^ r8) << 4);
    }
    const int zcols = p.N >> 3;
    uint32_t it = 0, tile_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_it) {
      int tile_m, tile_n;
      tile_coords(tile, p.mtiles, p.ntiles, &tile_m, &tile_n);
      const int m0 = tile_m * (128 * MH);
      const int n0 = tile_n * kBN;
      const int nA = n0 + col_local;
      const bool vA = nA < p.N;
      const uint32_t zshift = awq_slot_shift(static_cast<uint32_t>(nA & 7));

      auto load_sz = [&](int ks, uint32_t& sA, uint32_t& zA) {
        const int grp = (ks * kBK + hh * 32) / p.group_size;     // this thread's 32 k of the stage
        sA = vA ? __ldg(p.scales + static_cast<size_t>(grp) * p.N + nA) : 0u;
        zA = vA ? __ldg(p.qzeros + static_cast<size_t>(grp) * zcols + (nA >> 3)) : 0u;
      };
      uint32_t sA, zA, sA_n = 0, zA_n = 0;
      load_sz(0, sA, zA);

      for (int ks = 0; ks < nks; ++ks, ++it) {
        const int st = it % NT, sb = it % NB;
        const uint32_t ph = (it / NT) & 1u, phb = (it / NB) & 1u;
        const bool group_changes = (ks + 1 < nks) && (((ks + 1) * kBK) % p.group_size == 0);
        if (group_changes) load_sz(ks + 1, sA_n, zA_n);
        if (!mbar_wait(bar_full_tma(st), ph, abort_flag, 5)) { ok = false; break; }

        const unsigned char* raw = base_ptr + (raw_addr(st) - base);
        unsigned char* bst = base_ptr + (b_addr(sb) - base);
        const uint4 r0 = *reinterpret_cast<const uint4*>(raw + id * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty_tma(st));          // packed weights of this stage are in registers
        if (!mbar_wait(bar_empty_b(sb), phb ^ 1u, abort_flag, 7)) { ok = false; break; }
        {
          const ZeroPair zp = make_zero_pair((zA >> zshift) & 0xFu);
          const uint32_t s2 = sA * 0x00010001u;
          const uint32_t w[4] = {r0.x, r0.y, r0.z, r0.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t o[4];
            dequant_word(w[i], zp, s2, o);
            *reinterpret_cast<uint4*>(bst + boff[i]) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full_b(sb));
        if (group_changes) { sA = sA_n; zA = zA_n; }
      }
      if (!ok) break;

      // ------------------------------ epilogue --------------------------------
      if (!mbar_wait(bar_acc_full, tile_it & 1u, abort_flag, 6)) { ok = false; break; }
      tcgen05_fence_after();
      const bool has_bias = p.epi.bias != nullptr;
      const bool plain = !p.epi.gated && p.epi.residual == nullptr;
#pragma unroll 1
      for (int h = 0; h < MH; ++h) {
        const int row = m0 + h * 128 + lane_q * 32 + lane;
#pragma unroll 1
        for (int chunk = 0; chunk < 2; ++chunk) {
          const int col0 = n0 + col_quarter * 64 + chunk * 32;
          uint32_t v[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_q * 32) << 16) +
                                 static_cast<uint32_t>(h * 256 + col_quarter * 64 + chunk * 32);
          tcgen05_ld_32x32b_x32(taddr, v);   // whole warp, even if its rows are past M
          tcgen05_wait_ld();
          if (row < p.M) {
            uint16_t* yrow = p.y + static_cast<size_t>(row) * p.N;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int col = col0 + q * 8;
              if (col < p.N) {
                uint32_t b2[4] = {0u, 0u, 0u, 0u};
                if (has_bias) {
                  const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.epi.bias + col));
                  b2[0] = bv.x; b2[1] = bv.y; b2[2] = bv.z; b2[3] = bv.w;
                }
                uint4 out;
                out.x = cvt_pack_bias(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]), b2[0], has_bias);
                out.y = cvt_pack_bias(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]), b2[1], has_bias);
                out.z = cvt_pack_bias(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]), b2[2], has_bias);
                out.w = cvt_pack_bias(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]), b2[3], has_bias);
                if (plain) {
                  *reinterpret_cast<uint4*>(yrow + col) = out;
                } else {
                  const uint32_t words[4] = {out.x, out.y, out.z, out.w};
                  epilogue_finish_words<4>(p.y, p.epi, row, p.N, col, words);
                }
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(Cfg::kTmemCols))
                 : "memory");
  }
  if (tid == 0 && s_abort != 0 && p.status != nullptr) atomicCAS(p.status, 0u, static_cast<unsigned>(s_abort));
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static EncodeTiledFn g_encode = nullptr;

int get_encode(EncodeTiledFn* out) {
  EncodeTiledFn fn = __atomic_load_n(&g_encode, __ATOMIC_ACQUIRE);
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    AWQ_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !sym) return cuda_fail(cudaErrorNotSupported);
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    __atomic_store_n(&g_encode, fn, __ATOMIC_RELEASE);
  }
  *out = fn;
  return AWQ_B200_OK;
}

template <int MH>
static int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, const GemmParams& p, int sm_count,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<MH>;
  AWQ_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<MH>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  const int tiles = p.mtiles * p.ntiles;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_kernel<MH><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(mx, mw, p);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

// Weights-in-tensor-memory kernel (awq_wtm.cu).
size_t wtm_workspace_bytes(int sm_count);

// variant: 0 = pick by the cost table, 1 = dequantised weights in shared memory (this file)
int gemm_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                  void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream, int variant) {
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

  // Five tile shapes are available: the weights-in-tensor-memory kernel with 64 / 128 / 192 activation
  // rows per tile, and this file's kernel (dequantised weights in shared memory) with 128 / 256 rows.
  // Cost = waves of CTA tiles x measured time of one 64-k stage of that tile shape (microseconds on
  // B200); all variants give identical bits, so the choice only affects speed.
  const int ntiles = (N + kBN - 1) / kBN;
  auto waves = [&](int rows) {
    const long long t = static_cast<long long>((M + rows - 1) / rows) * ntiles;
    return static_cast<double>((t + di.sm_count - 1) / di.sm_count);
  };
  // The tensor-memory variant shares a partial last wave between all SMs when the workspace allows
  // (see awq_wtm.cu): its cost then grows with the exact tile count, plus a little for the fix-up.
  const bool can_split = workspace_bytes >= wtm_workspace_bytes(di.sm_count);
  auto waves_wtm = [&](int rows) {
    const long long t = static_cast<long long>((M + rows - 1) / rows) * ntiles;
    // the split is taken when the idle share of the last (or only) wave is worth more than ~35 us
    const double idle_us = (t % di.sm_count) ? (1.0 - static_cast<double>(t % di.sm_count) / di.sm_count) * (K / 64) * 0.6 : 0.0;
    if (!can_split || idle_us <= 35.0) return waves(rows);
    return static_cast<double>(t) / di.sm_count + 0.08;
  };
  const double c_wtm64 = waves_wtm(64) * 0.43, c_wtm128 = waves_wtm(128) * 0.52, c_wtm192 = waves_wtm(192) * 0.64;
  const double c_smem1 = waves(128) * 0.78, c_smem2 = waves(256) * 1.00;
  int MH = (M > 128 && c_smem2 <= c_smem1) ? 2 : 1;
  if (variant == 0) {
    const double c_smem = MH == 2 ? c_smem2 : c_smem1;
    double c_w = c_wtm192;
    int mt = 192;
    if (c_wtm128 < c_w) { c_w = c_wtm128; mt = 128; }
    if (c_wtm64 < c_w) { c_w = c_wtm64; mt = 64; }
    if (c_w <= c_smem)
      return wtm_dispatch(x, packed, scales, qzeros, epi, y, M, K, N, group_size, workspace, workspace_bytes, stream, mt);
  }

  CUtensorMap mx, mw;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t box[2] = {kBK, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }
  {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K / kBlockK)};
    const cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(N) * 64};
    const cuuint32_t box[3] = {32, kBN, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(packed), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  }

  GemmParams p;
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.epi = epi;
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  p.M = M; p.K = K; p.N = N;
  p.group_size = group_size;
  p.ntiles = ntiles;
  p.mtiles = (M + 128 * MH - 1) / (128 * MH);
  return MH == 2 ? launch_gemm<2>(mx, mw, p, di.sm_count, stream) : launch_gemm<1>(mx, mw, p, di.sm_count, stream);
}

}  // namespace awq

using namespace awq;

extern "C" {

// 256 bytes (the status word) are enough for a correct result; with the full size the tensor-memory
// variant may cut the tiles of a partial last wave along k and share them between all SMs.
size_t awq_b200_gemm_workspace_bytes(int M, int K, int N) {
  (void)M; (void)K; (void)N;
  DeviceInfo di;
  int sm = 148;
  if (device_info(&di) == AWQ_B200_OK) sm = di.sm_count;
  return wtm_workspace_bytes(sm);
}

int awq_b200_gemm(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                  void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                  awq_b200_stream_t stream) {
  return gemm_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream), 0);
}

// Tuning hook: awq_b200_gemm restricted to the kernel that stages the dequantised weights in shared memory.
int awq_b200_gemm_smem(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const void* bias,
                       void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                       awq_b200_stream_t stream) {
  return gemm_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream), 1);
}

}  // extern "C"
