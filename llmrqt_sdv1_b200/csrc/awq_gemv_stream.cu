// Decode path for large weight matrices: the split-K W4A16 GEMV as a persistent, evenly balanced
// stream ("stream-K").
//
// The arithmetic, the packed layout and the roles inside a CTA are those of gemv_kernel (W compute
// warps as a CW x KW grid, one warp that only issues bulk copies, weights as the mma A operand,
// fp32 scale / zero point per 128-k block).  What differs is how work reaches the CTAs:
//
//   unit      = KW consecutive 128-k blocks of one column group.  A column group is CW x 4 column
//               tiles wide whatever NTW is (with NTW = 2 a CTA walks a segment twice, once per half
//               of the group), so the k ranges that are added separately, and with them the result
//               bits, do not depend on the row count that picks NTW.  A column group has
//               ipc = ceil(nblk / KW) units; U = ncol * ipc in total.
//   CTA b     = units [b*U/G, (b+1)*U/G) of the flattened (column group, iteration) sequence, with
//               G = resident CTAs of the device.  Every CTA streams the same number of units (+-1)
//               through ONE copy pipeline that never drains between column groups: while the
//               compute warps finish a column group (reduction, output), the producer is already
//               filling the ring with the next one's weights.
//   segment   = the units of one column group inside one CTA.  A column group that lies inside one
//               CTA is written straight to y; one that straddles CTAs is written as fp32 partials,
//               one slot per contributing CTA, and the last contributor to arrive adds the slots in
//               CTA order (= k order), so the result is deterministic and does not depend on M.
//
// Compared with one CTA per (column group, k-split) this removes the pipeline fill and the
// reduction tail from the critical path of every CTA but the first, and the wave quantisation of
// grids that are not a multiple of the resident CTA count.
#include "awq_gemv_common.cuh"

namespace awq {

struct GemvStreamParams {
  GemvParams g;        // pointers, M/K/N, group_blocks, nblk, ntiles (bps, S, cluster unused)
  int ncol;            // column groups
  int ipc;             // units per column group
  long long units;     // ncol * ipc
};
struct GemvStreamParamsFused : GemvStreamParams {
  GemvFusion fusion;
};
template <bool FUSED> struct GemvStreamParamsOf { using type = GemvStreamParams; };
template <> struct GemvStreamParamsOf<true> { using type = GemvStreamParamsFused; };

template <int W>
__device__ __forceinline__ void compute_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
}

// FUSED = false compiles the residual / gated parts of the epilogue out (bias only).
template <int NTW, int MT, int KW, int W, bool FUSED>
__global__ void __launch_bounds__((W + 1) * 32, W == 8 ? 2 : 1) gemv_stream_kernel(const typename GemvStreamParamsOf<FUSED>::type sp) {
  const GemvParams& p = sp.g;
  const GemvFusion* fusion = nullptr;   // compile-time null in the unfused variants
  if constexpr (FUSED) fusion = &sp.fusion;
  const bool gated = fusion != nullptr && fusion->gated != 0;
  constexpr int kComputeThreads = W * 32;
  static_assert(NTW == 2 || NTW == 4, "column tiles are processed in pairs");
  static_assert(W == 8 || W == 16, "8 or 16 compute warps");
  static_assert(KW >= 1 && KW <= W && (W % KW) == 0 && (KW & (KW - 1)) == 0, "KW divides the compute warps");
  constexpr int NP = NTW / 2;
  constexpr int MH = MT / 8;
  constexpr int CW = W / KW;
  constexpr int kCtaTiles = CW * NTW;       // column tiles in flight per pass
  constexpr int kCtaCols = kCtaTiles * 8;
  constexpr int kPasses = 4 / NTW;          // passes over a segment: the column group is CW x 4 tiles
  constexpr int kGroupTiles = CW * 4;
  constexpr int kSubWeights = kCtaTiles * 512;
  constexpr int kSubScaleOff = kSubWeights;
  constexpr int kSubZeroOff = kSubScaleOff + kCtaTiles * 16;
  constexpr int kSubBytes = kSubWeights + kCtaTiles * 32;
  constexpr int kStageBytes = KW * kSubBytes;
  constexpr int ST = gemv_stages(NTW, W);
  constexpr int kRedFloats = (KW > 1 ? KW : 0) * MT * kCtaCols;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_last;
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const bool is_producer = (warp == W);
  const int cw = warp % CW, kw = (warp / CW) % KW;

  // Shared memory: [ring: ST stages][reduction buffer: KW x MT x kCtaCols floats][mbarriers]
  unsigned char* ring = smem;
  float* red_k = reinterpret_cast<float*>(smem + ST * kStageBytes);
  const uint32_t bar_base = smem_u32(smem + ST * kStageBytes + kRedFloats * 4);
  auto bar_full = [&](int st) { return bar_base + 8u * st; };
  auto bar_empty = [&](int st) { return bar_base + 8u * (ST + st); };
  volatile int* abort_flag = &s_abort;

  const long long U = sp.units, G = gridDim.x;
  const long long u0 = stream_first_unit(blockIdx.x, U, G), u1 = stream_first_unit(blockIdx.x + 1, U, G);
  const int ipc = sp.ipc;
  const int zcols = p.N >> 3;
  const size_t block_stride_u4 = static_cast<size_t>(p.N) * 4;

  // ------------------------------------------------------------------ producer
  // Stage gs (counted from this CTA's first unit) holds unit u0 + gs.  The whole warp runs the
  // loop; lane j issues the three copies of block j of the unit.
  int issued = 0;
  auto issue_stage = [&](int cg, int pass, int it, int gs) {
    const int cta_tile0 = cg * kGroupTiles + pass * kCtaTiles;
    const uint32_t valid_tiles = static_cast<uint32_t>(max(0, min(kCtaTiles, p.ntiles - cta_tile0)));
    const bool zeros_by_copy = ((p.N & 31) == 0) && ((valid_tiles & 3u) == 0u);
    const uint32_t sub_tx = valid_tiles * (512u + 16u + (zeros_by_copy ? 4u : 0u));
    const int st = gs % ST;
    const int nblocks = min(KW, p.nblk - it * KW);
    const uint32_t bar = bar_full(st);
    if (valid_tiles == 0u) {          // a pass entirely beyond the last column: nothing to copy
      if (lane == 0) mbar_arrive(bar);
      return;
    }
    if (lane == 0) mbar_expect_tx(bar, sub_tx * static_cast<uint32_t>(nblocks));
    if (lane < nblocks) {
      const int bl = it * KW + lane;
      const uint32_t dst = smem_u32(ring + st * kStageBytes + lane * kSubBytes);
      const int grp = p.group_blocks == 1 ? bl : bl / p.group_blocks;
      bulk_load(dst, p.wp + static_cast<size_t>(bl) * block_stride_u4 + static_cast<size_t>(cta_tile0) * 32,
                valid_tiles * 512u, bar);
      bulk_load(dst + kSubScaleOff, p.scales + static_cast<size_t>(grp) * p.N + static_cast<size_t>(cta_tile0) * 8,
                valid_tiles * 16u, bar);
      if (zeros_by_copy)
        bulk_load(dst + kSubZeroOff, p.qzeros + static_cast<size_t>(grp) * zcols + cta_tile0, valid_tiles * 4u, bar);
    }
  };
  // Producer cursor over this CTA's stages: segments in unit order, inside a segment pass-major.
  long long pu = u0;                   // first unit of the current segment
  int p_cg = 0, p_begin = 0, p_end = 0, p_pass = 0, p_it = 0;
  auto open_segment = [&]() {
    p_cg = static_cast<int>(pu / ipc);
    p_begin = static_cast<int>(pu - static_cast<long long>(p_cg) * ipc);
    p_end = static_cast<int>(min(static_cast<long long>(ipc), p_begin + (u1 - pu)));
    p_pass = 0;
    p_it = p_begin;
  };
  auto issue_next = [&](int gs) {
    issue_stage(p_cg, p_pass, p_it, gs);
    if (++p_it == p_end) {
      p_it = p_begin;
      if (++p_pass == kPasses) {
        pu += p_end - p_begin;
        if (pu < u1) open_segment();
      }
    }
  };

  const int my_stages = static_cast<int>(u1 - u0) * kPasses;
  if (is_producer) {
    if (lane == 0) s_abort = 0;
    if (lane < ST) {
      mbar_init(bar_full(lane), 1);
      mbar_init(bar_empty(lane), W);
      mbar_fence_init();
    }
    __syncwarp();
    if (my_stages > 0) open_segment();
#pragma unroll
    for (int gs = 0; gs < ST; ++gs) {
      if (gs < my_stages) {
        issue_next(gs);
        issued = gs + 1;
      }
    }
  }
  // Everything requested so far is constant data.  Let the next kernel of the stream start its own
  // prefetch, and wait for the previous one before touching activations, outputs or the workspace
  // (both are no-ops unless the launch asked for programmatic dependent launch).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();   // mbarrier initialisation visible to every warp

  if (is_producer) {
    for (int gs = ST; gs < my_stages; ++gs) {
      if (!mbar_wait(bar_empty(gs % ST), static_cast<uint32_t>(gs / ST - 1) & 1u, abort_flag, 2)) break;
      issue_next(gs);
      issued = gs + 1;
    }
  } else {
    // ---------------------------------------------------------------- compute warps
    // After a failed wait a warp stops computing but keeps walking its segments, so that every
    // compute warp still meets the others at each segment's named barriers.
    bool ok = true;
    int gs = 0;
    long long u = u0;
    while (u < u1) {
      const int cg = static_cast<int>(u / ipc);
      const int it_begin = static_cast<int>(u - static_cast<long long>(cg) * ipc);
      const int it_end = static_cast<int>(min(static_cast<long long>(ipc), it_begin + (u1 - u)));
      // Contributors of this column group: the CTAs that own its first and last unit, and all between.
      const long long cg_u0 = static_cast<long long>(cg) * ipc;
      const int c_first = stream_cta_of(cg_u0, U, G);
      const int c_last = stream_cta_of(cg_u0 + ipc - 1, U, G);
      const int nc = c_last - c_first + 1;
      const int slot = static_cast<int>(blockIdx.x) - c_first;
      const bool direct = (nc == 1) && !gated;   // a gated epilogue pairs columns in the reduction below
      for (int pass = 0; pass < kPasses; ++pass) {
        const int cta_tile0 = cg * kGroupTiles + pass * kCtaTiles;
        const int tile0 = cta_tile0 + cw * NTW;
        const uint32_t valid_tiles = static_cast<uint32_t>(max(0, min(kCtaTiles, p.ntiles - cta_tile0)));
        const bool zeros_by_copy = ((p.N & 31) == 0) && ((valid_tiles & 3u) == 0u);

        // Activations go straight from global memory (L1/L2 resident) to the mma B fragments: lane
        // (g, c) needs row 8*mh + g, k = 32c .. 32c+31 of each block, i.e. 64 contiguous bytes.
        const uint16_t* xlane[MH];
        bool xvalid[MH];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
          const int m = mh * 8 + g;
          xvalid[mh] = m < p.M;
          xlane[mh] = p.x + static_cast<size_t>(xvalid[mh] ? m : 0) * p.K + c * 32;
        }
        auto load_x = [&](int bl, uint4 (&xv)[MH][4]) {
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              xv[mh][i] = make_uint4(0u, 0u, 0u, 0u);
              if (xvalid[mh] && bl < p.nblk)
                xv[mh][i] = __ldg(reinterpret_cast<const uint4*>(xlane[mh] + static_cast<size_t>(bl) * kBlockK + i * 8));
            }
          }
        };
        constexpr bool kPrefetchX = (MH == 1);   // double-buffer the fragments when registers allow
        uint4 xnext[MH][4];
        if (kPrefetchX) load_x(it_begin * KW + kw, xnext);

        float acc[MH][NP][4];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh)
#pragma unroll
          for (int q = 0; q < NP; ++q) acc[mh][q][0] = acc[mh][q][1] = acc[mh][q][2] = acc[mh][q][3] = 0.f;

        for (int it = it_begin; it < it_end; ++it, ++gs) {
          const int st = gs % ST;
          const uint32_t ph = static_cast<uint32_t>(gs / ST) & 1u;
          const int bl = it * KW + kw;               // this warp's block in this unit
          if (ok && !mbar_wait(bar_full(st), ph, abort_flag, 1)) ok = false;
          if (!ok) continue;
          uint4 wv[NTW];
          float sc[NTW], zp[NTW];
          if (bl < p.nblk && valid_tiles != 0u) {
            const unsigned char* sub = ring + st * kStageBytes + kw * kSubBytes;
            const unsigned char* src = sub + (cw * NTW) * 512 + lane * 16;
#pragma unroll
            for (int t = 0; t < NTW; ++t) wv[t] = *reinterpret_cast<const uint4*>(src + t * 512);
            const unsigned short* ssrc = reinterpret_cast<const unsigned short*>(sub + kSubScaleOff) + (cw * NTW) * 8 + g;
            const uint32_t* zsrc = reinterpret_cast<const uint32_t*>(sub + kSubZeroOff) + cw * NTW;
#pragma unroll
            for (int t = 0; t < NTW; ++t) {
              sc[t] = __half2float(__ushort_as_half(ssrc[t * 8]));
              uint32_t zw;
              if (zeros_by_copy) zw = zsrc[t];
              else zw = __ldg(p.qzeros + static_cast<size_t>(bl / p.group_blocks) * zcols + min(tile0 + t, p.ntiles - 1));
              zp[t] = small_uint_to_float((zw >> awq_slot_shift(g)) & 0xFu);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty(st));
          if (bl >= p.nblk || valid_tiles == 0u) continue;

          uint4 xv[MH][4];
          float4 T[MH];
          if (kPrefetchX) {
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[0][i] = xnext[0][i];
            load_x(bl + KW, xnext);
          } else {
            load_x(bl, xv);
          }
          gemv_block_sums<MH>(xv, T);
          gemv_block_pairs<NTW, MH>(wv, sc, zp, xv, T, acc);
        }

        // ---- segment epilogue (one per pass) ---------------------------------------------------
        // Where one finished element of this segment goes: y, or this CTA's slot of the partials.
        auto emit = [&](int m, int nl, float v) {
          const int n = cta_tile0 * 8 + nl;
          if (n >= p.N) return;
          if (direct) variant_store_one(p, fusion, m, n, v);
          else __stcg(p.partial + (static_cast<size_t>(slot) * p.M + m) * p.N + n, v);
        };
        // A compute thread holds rows m = 8*mh + 2c, +1 of columns n and n + 8 of each of its pairs.
        if (KW > 1) compute_warps_sync<W>();   // the previous segment's reduction has been read
#pragma unroll
        for (int q = 0; q < NP; ++q) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int nl = (cw * NTW + 2 * q + half) * 8 + g;
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int m = mh * 8 + 2 * c + e;
                if (m >= p.M) continue;
                const float v = acc[mh][q][half * 2 + e];
                if (KW == 1) emit(m, nl, v);
                else red_k[(kw * p.M + m) * kCtaCols + nl] = v;
              }
            }
          }
        }
        if (KW > 1) {
          // The KW warps of a column group add their sums in kw order.
          compute_warps_sync<W>();
          for (int e = tid; e < p.M * kCtaCols; e += kComputeThreads) {
            float v = red_k[e];
#pragma unroll
            for (int j = 1; j < KW; ++j) v += red_k[j * p.M * kCtaCols + e];
            emit(e / kCtaCols, e % kCtaCols, v);
          }
        }
        if (!direct) {
          __threadfence();
          compute_warps_sync<W>();
          if (tid == 0) {
            const unsigned prev = atomicAdd(&p.counters[cg * kPasses + pass], 1u);
            const int last = (prev == static_cast<unsigned>(nc - 1));
            if (last) p.counters[cg * kPasses + pass] = 0u;   // every contributor has arrived: leave the counter clean
            s_last = last;
          }
          compute_warps_sync<W>();
          if (s_last) {
            __threadfence();
            // The last contributor adds the nc slots in CTA order, which is k order.
            const int col0 = cta_tile0 * 8;
            const int ncols = min(kCtaCols, p.N - col0);
            const int pairs = ncols >> 1;
            const size_t slot_stride = static_cast<size_t>(p.M) * p.N;
            for (int i = tid; i < p.M * pairs; i += kComputeThreads) {
              const int row = i / pairs;
              const int col = col0 + 2 * (i - row * pairs);
              const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
              const float2 sum = sum_partial_slots(src, slot_stride, nc);
              variant_store_pair(p, fusion, row, col, sum.x, sum.y);
            }
          }
        }
      }
      u += it_end - it_begin;
    }
  }

  __syncthreads();
  if (s_abort != 0) {
    // A wait expired.  Let this CTA's outstanding copies land (bounded) before shared memory is
    // released and record the failure: the output of this call is invalid and the arrival
    // counters must be zeroed again before the workspace is reused.
    if (is_producer && lane == 0) {
      for (int gs = max(0, issued - ST); gs < issued; ++gs)
        mbar_wait_timed(bar_full(gs % ST), static_cast<uint32_t>(gs / ST) & 1u);
      if (p.status != nullptr) atomicCAS(p.status, 0u, static_cast<unsigned>(s_abort));
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static int stream_grid(int w, int sm_count, long long units) {
  const long long resident = static_cast<long long>(w == 8 ? 2 : 1) * sm_count;
  return static_cast<int>(units < resident ? units : resident);
}

// Largest number of CTAs that share one column group (= partial slots needed) for this decomposition.
int gemv_stream_slots(int K, int N, int ntw, int w, int kw, int sm_count) {
  const int nblk = K / kBlockK, ntiles = N / 8;
  (void)ntw;                                 // the column group is (w / kw) x 4 tiles whatever ntw is
  const int group_tiles = (w / kw) * 4;
  const int ncol = (ntiles + group_tiles - 1) / group_tiles;
  const int ipc = (nblk + kw - 1) / kw;
  const long long U = static_cast<long long>(ncol) * ipc;
  const long long G = stream_grid(w, sm_count, U);
  int worst = 1;
  for (int cg = 0; cg < ncol; ++cg) {
    const long long a = static_cast<long long>(cg) * ipc;
    const int nc = stream_cta_of(a + ipc - 1, U, G) - stream_cta_of(a, U, G) + 1;
    if (nc > worst) worst = nc;
  }
  return worst;
}

template <int NTW, int MT, int KW, int W, bool FUSED>
static int launch_stream(const GemvStreamParams& sp_plain, const GemvFusion& fusion, int grid, int max_smem_optin,
                         cudaStream_t stream, bool overlap_previous) {
  typename GemvStreamParamsOf<FUSED>::type sp;
  static_cast<GemvStreamParams&>(sp) = sp_plain;
  if constexpr (FUSED) sp.fusion = fusion;
  constexpr int ST = gemv_stages(NTW, W);
  constexpr int kCtaCols = (W / KW) * NTW * 8;
  const size_t smem = static_cast<size_t>(ST) * W * NTW * (512 + 32) + (KW > 1 ? KW : 0) * MT * kCtaCols * 4 + 2 * ST * 8;
  if (smem > static_cast<size_t>(max_smem_optin)) return AWQ_B200_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    AWQ_CUDA_TRY(cudaFuncSetAttribute(gemv_stream_kernel<NTW, MT, KW, W, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((W + 1) * 32);
  cfg.dynamicSmemBytes = smem;
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
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<NTW, MT, KW, W, FUSED>, sp));
  return AWQ_B200_OK;
}

// Launches the streaming kernel for a decomposition (ntw, w, kw) the caller has validated.  `base`
// carries pointers and sizes; partial / counters must be set when gemv_stream_slots(...) > 1.
int gemv_stream_launch(const GemvParams& base, const GemvFusion& fusion, int ntw, int w, int kw, int sm_count,
                       int max_smem_optin, cudaStream_t stream, bool overlap_previous) {
  GemvStreamParams sp;
  sp.g = base;
  const int group_tiles = (w / kw) * 4;
  sp.ncol = (base.ntiles + group_tiles - 1) / group_tiles;
  if (sp.ncol * (4 / ntw) > kGemvMaxCounters - 1) return AWQ_B200_ERR_TOO_LARGE;
  sp.ipc = (base.nblk + kw - 1) / kw;
  sp.units = static_cast<long long>(sp.ncol) * sp.ipc;
  const int grid = stream_grid(w, sm_count, sp.units);
  const bool wide = base.M > 8;
  const bool fused = fusion.gated || fusion.residual != nullptr;
#define AWQ_STREAM_CASE(NTW_, KW_, W_)                                                                \
  if (ntw == NTW_ && kw == KW_ && w == W_)                                                            \
    return fused ? (wide ? launch_stream<NTW_, 16, KW_, W_, true>(sp, fusion, grid, max_smem_optin, stream, overlap_previous)   \
                         : launch_stream<NTW_, 8, KW_, W_, true>(sp, fusion, grid, max_smem_optin, stream, overlap_previous))   \
                 : (wide ? launch_stream<NTW_, 16, KW_, W_, false>(sp, fusion, grid, max_smem_optin, stream, overlap_previous)  \
                         : launch_stream<NTW_, 8, KW_, W_, false>(sp, fusion, grid, max_smem_optin, stream, overlap_previous));
  AWQ_STREAM_CASE(2, 1, 8) AWQ_STREAM_CASE(2, 2, 8) AWQ_STREAM_CASE(2, 4, 8) AWQ_STREAM_CASE(2, 8, 8)
  AWQ_STREAM_CASE(4, 1, 8) AWQ_STREAM_CASE(4, 2, 8) AWQ_STREAM_CASE(4, 4, 8) AWQ_STREAM_CASE(4, 8, 8)
  AWQ_STREAM_CASE(2, 4, 16) AWQ_STREAM_CASE(2, 8, 16) AWQ_STREAM_CASE(2, 16, 16)
  AWQ_STREAM_CASE(4, 4, 16) AWQ_STREAM_CASE(4, 8, 16) AWQ_STREAM_CASE(4, 16, 16)
  return AWQ_B200_ERR_SHAPE;
#undef AWQ_STREAM_CASE
}

}  // namespace awq
