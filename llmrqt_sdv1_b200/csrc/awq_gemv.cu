// Decode path: split-K W4A16 GEMV for 1 <= M <= 64 rows (8 rows per CTA).
//
// One pass over the packed weights serves 8 rows; more rows run as more CTAs per (column group, split), which
// read the same weights at about the same time (L2 hits) and unpack them once each.  Work unit = one 128-k
// block x one tile of 8 output columns = 512 contiguous bytes, read by a warp
// as one 128-bit load per lane.  Lane (g = lane / 4, c = lane % 4) owns column
// 8*tile + g and the four words 4c..4c+3 of that column (32 consecutive k).
// Two adjacent tiles form the 16 rows of an mma.sync m16n8k16 A operand; the
// nibbles go to the tensor core as unscaled codes and scale / zero point are
// applied in fp32 once per 128-k block, which keeps the instruction count per
// byte low enough for the kernel to be bound by HBM rather than by issue slots.
// k is split over gridDim.y; each split writes fp32 partials to the workspace
// and the last CTA to arrive for a column range adds them in split order, so
// results are deterministic and a row's value does not depend on how many rows
// the call has.
#include "awq_gemv_common.cuh"

namespace awq {

// The W compute warps form a CW x KW grid (CW * KW = W): warp (cw, kw) owns NTW column tiles
// (NTW/2 pairs of 16 columns) and every KW-th 128-k block of this CTA's k-range.  MT = 8 or 16 rows.
//
// Arithmetic per 128-k block b, column n, row m (all fp32 after the tensor core):
//   y[m,n] += s[b,n] * ( sum_k x[m,k] * code[k,n]  -  z[b,n] * sum_k x[m,k] )
// The 16 columns of a pair are the rows of the mma A operand (the weights), the activations are the
// B operand (8 rows of x per mma), so one m16n8k16 covers 16 columns x 16 k.  The activation sums
// per block and row come from the tensor core as well.  Sums are added in a fixed order: a warp's
// blocks in k order, then the KW warps of a column group in kw order (shared memory), then the
// grid-level splits in split order (cluster shared memory or the global workspace).
// FUSED = false compiles the residual / gated parts of the epilogue out (bias only).
// ROW_HALVES = true serves more than MT rows with gridDim.z CTAs per (column group, split).
template <int NTW, int MT, int KW, int W, bool FUSED, bool ROW_HALVES>
__global__ void __launch_bounds__((W + 1) * 32, W == 8 ? 2 : 1) gemv_kernel(const typename GemvParamsOf<FUSED>::type p) {
  const GemvFusion* fusion = nullptr;   // compile-time null in the unfused variants
  if constexpr (FUSED) fusion = &p.fusion;
  const bool gated = fusion != nullptr && fusion->gated != 0;
  constexpr int kGemvWarps = W;
  constexpr int kGemvThreads = (W + 1) * 32;
  static_assert(NTW == 2 || NTW == 4, "column tiles are processed in pairs");
  static_assert(W == 8 || W == 16, "8 or 16 compute warps");
  static_assert(KW >= 1 && KW <= W && (W % KW) == 0 && (KW & (KW - 1)) == 0, "KW divides the compute warps");
  constexpr int NP = NTW / 2;              // pairs per warp
  constexpr int MH = MT / 8;               // row halves
  constexpr int CW = kGemvWarps / KW;      // column groups per CTA
  constexpr int kCtaTiles = CW * NTW;      // 8-column tiles per CTA
  constexpr int kCtaCols = kCtaTiles * 8;
  constexpr int kSubWeights = kCtaTiles * 512;            // one block of this CTA's columns
  constexpr int kSubScaleOff = kSubWeights;               // then kCtaTiles * 8 fp16 scales
  constexpr int kSubZeroOff = kSubScaleOff + kCtaTiles * 16;
  constexpr int kSubBytes = kSubWeights + kCtaTiles * 32; // one block: weights, scales, zero words (padded)
  constexpr int kStageBytes = KW * kSubBytes;             // one pipeline stage: KW consecutive blocks
  constexpr int ST = gemv_stages(NTW, W);
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_last;
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = blockIdx.y;
  // More than MT rows: gridDim.z CTAs per (column group, split), each with its own MT rows.  The halves run
  // side by side and read the same weights at about the same time, so the second read is an L2 hit.
  const int row0 = ROW_HALVES ? blockIdx.z * MT : 0;
  const int rows = ROW_HALVES ? min(p.M - row0, MT) : p.M;      // rows of this CTA
  const bool is_producer = (warp == kGemvWarps);
  const int cw = warp % CW, kw = (warp / CW) % KW;
  const int b0 = split * p.bps;
  const int nb = min(p.bps, p.nblk - b0);        // blocks of this split
  const int nit = (nb + KW - 1) / KW;            // pipeline iterations (KW blocks each)

  // Shared memory: [ring: ST stages][mbarriers]; the ring is reused for the reductions at the end.
  unsigned char* ring = smem;
  const uint32_t bar_base = smem_u32(ring + ST * kStageBytes);
  auto bar_full = [&](int st) { return bar_base + 8u * st; };
  auto bar_empty = [&](int st) { return bar_base + 8u * (ST + st); };
  volatile int* abort_flag = &s_abort;

  const int cta_tile0 = blockIdx.x * kCtaTiles;
  const int tile0 = cta_tile0 + cw * NTW;
  const int zcols = p.N >> 3;
  const uint32_t valid_tiles = static_cast<uint32_t>(min(kCtaTiles, p.ntiles - cta_tile0));
  const uint4* wsrc = p.wp + (static_cast<size_t>(b0) * p.N) * 4 + static_cast<size_t>(cta_tile0) * 32;
  const size_t block_stride_u4 = static_cast<size_t>(p.N) * 4;
  // qzeros rows can be bulk-copied only if every row segment is 16-byte aligned and sized.
  const bool zeros_by_copy = ((p.N & 31) == 0) && ((valid_tiles & 3u) == 0u);
  const uint32_t sub_tx = valid_tiles * (512u + 16u + (zeros_by_copy ? 4u : 0u));
  // One stage = the packed weights, scales and zero words of KW consecutive blocks.  The whole
  // producer warp calls this: lane j issues the copies of block j, so a stage costs three copy
  // instructions however many blocks it has (a single thread issuing them one after another needs
  // longer than the copies take).
  auto issue_stage = [&](int it) {
    const int st = it % ST;
    const int nblocks = min(KW, nb - it * KW);
    const uint32_t bar = bar_full(st);
    if (lane == 0) mbar_expect_tx(bar, sub_tx * static_cast<uint32_t>(nblocks));
    if (lane < nblocks) {
      const int bl = it * KW + lane;
      const uint32_t dst = smem_u32(ring + st * kStageBytes + lane * kSubBytes);
      const int grp = p.group_blocks == 1 ? (b0 + bl) : (b0 + bl) / p.group_blocks;
      bulk_load(dst, wsrc + static_cast<size_t>(bl) * block_stride_u4, valid_tiles * 512u, bar);
      bulk_load(dst + kSubScaleOff, p.scales + static_cast<size_t>(grp) * p.N + static_cast<size_t>(cta_tile0) * 8,
                valid_tiles * 16u, bar);
      if (zeros_by_copy)
        bulk_load(dst + kSubZeroOff, p.qzeros + static_cast<size_t>(grp) * zcols + cta_tile0, valid_tiles * 4u, bar);
    }
  };

  int issued = 0;   // stages whose copies have been started (meaningful in the producer warp only)
  if (is_producer) {
    if (lane == 0) s_abort = 0;
    if (lane < ST) {
      mbar_init(bar_full(lane), 1);
      mbar_init(bar_empty(lane), kGemvWarps);
      mbar_fence_init();
    }
    __syncwarp();
#pragma unroll
    for (int st = 0; st < ST; ++st) {
      if (st < nit) {
        issue_stage(st);
        issued = st + 1;
      }
    }
  }
  // Everything requested so far is constant data.  Let the next kernel of the stream start its own
  // prefetch, and wait for the previous one before touching activations, outputs or the workspace
  // (both are no-ops unless the launch asked for programmatic dependent launch).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();   // mbarrier initialisation visible to every warp

  // Activations go straight from global memory (L1/L2 resident) to the mma B fragments: lane
  // (g, c) needs row 8*mh + g, k = 32c .. 32c+31 of each block, i.e. 64 contiguous bytes.
  const uint16_t* xlane[MH];
  bool xvalid[MH];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh) {
    const int m = mh * 8 + g;
    xvalid[mh] = m < rows;
    xlane[mh] = p.x + static_cast<size_t>(xvalid[mh] ? row0 + m : 0) * p.K + static_cast<size_t>(b0) * kBlockK + c * 32;
  }
  auto load_x = [&](int bl, uint4 (&xv)[MH][4]) {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xv[mh][i] = make_uint4(0u, 0u, 0u, 0u);
        if (xvalid[mh] && bl < nb) xv[mh][i] = __ldg(reinterpret_cast<const uint4*>(xlane[mh] + bl * kBlockK + i * 8));
      }
    }
  };
  constexpr bool kPrefetchX = (MH == 1);   // double-buffer the fragments when registers allow
  uint4 xnext[MH][4];
  if (!is_producer && kPrefetchX) load_x(kw, xnext);

  float acc[MH][NP][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int q = 0; q < NP; ++q) acc[mh][q][0] = acc[mh][q][1] = acc[mh][q][2] = acc[mh][q][3] = 0.f;

  if (is_producer) {
    // Producer warp: refill a stage as soon as all compute warps have released it.
    for (int it = ST; it < nit; ++it) {
      if (!mbar_wait(bar_empty(it % ST), static_cast<uint32_t>(it / ST - 1) & 1u, abort_flag, 2)) break;
      issue_stage(it);
      issued = it + 1;
    }
  } else {
    for (int it = 0; it < nit; ++it) {
      const int st = it % ST;
      const uint32_t ph = static_cast<uint32_t>(it / ST) & 1u;
      const int bl = it * KW + kw;               // this warp's block in this iteration
      if (!mbar_wait(bar_full(st), ph, abort_flag, 1)) break;
      uint4 wv[NTW];
      float sc[NTW], zp[NTW];
      if (bl < nb) {
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
          else zw = __ldg(p.qzeros + static_cast<size_t>((b0 + bl) / p.group_blocks) * zcols +
                          min(tile0 + t, p.ntiles - 1));
          zp[t] = small_uint_to_float((zw >> awq_slot_shift(g)) & 0xFu);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty(st));
      if (bl >= nb) continue;

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
  }
  __syncthreads();
  if (s_abort != 0) {
    // A wait expired.  Let this CTA's outstanding copies land (bounded) before shared memory is
    // released, record the failure, and fall through: the output of this call is invalid.
    if (is_producer && lane == 0) {
      for (int it = max(0, issued - ST); it < issued; ++it)
        mbar_wait_timed(bar_full(it % ST), static_cast<uint32_t>(it / ST) & 1u);
      if (p.status != nullptr) atomicCAS(p.status, 0u, static_cast<unsigned>(s_abort));
    }
    __syncthreads();
  }

  // ---- epilogue -------------------------------------------------------------------------------
  // A compute thread holds rows m = 8*mh + 2c, +1 of columns n and n + 8 of each of its pairs.
  // A gated epilogue needs both columns of a pair in one thread: it always finishes through the partials.
  const bool direct = (p.S == 1) && !gated;
  const bool via_cluster = (p.cluster != 0);
  float* red_k = reinterpret_cast<float*>(ring);                 // [KW][M][kCtaCols]  (KW > 1 only)
  float* red = red_k + (KW > 1 ? KW * rows * kCtaCols : 0);       // [M][kCtaCols]      (cluster only)
  // Where one finished element of this CTA goes: y, the cluster buffer, or the global partials.
  auto emit = [&](int m, int nl, float v) {
    const int n = cta_tile0 * 8 + nl;
    if (n >= p.N) return;
    if (direct) variant_store_one(p, fusion, row0 + m, n, v);
    else if (via_cluster) red[m * kCtaCols + nl] = v;
    else __stcg(p.partial + (static_cast<size_t>(split) * p.M + row0 + m) * p.N + n, v);
  };
  if (!is_producer) {
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
            if (m >= rows) continue;
            const float v = acc[mh][q][half * 2 + e];
            if (KW == 1) emit(m, nl, v);
            else red_k[(kw * rows + m) * kCtaCols + nl] = v;
          }
        }
      }
    }
  }
  if (KW > 1) {
    // The KW warps of a column group add their sums in kw order.
    __syncthreads();
    for (int e = tid; e < rows * kCtaCols; e += kGemvThreads) {
      float v = red_k[e];
#pragma unroll
      for (int j = 1; j < KW; ++j) v += red_k[j * rows * kCtaCols + e];
      emit(e / kCtaCols, e % kCtaCols, v);
    }
  }
  if (direct) return;

  if (via_cluster) {
    // The S splits of this column range are the CTAs of one cluster (rank = split).  Each rank
    // adds, in split order, the S partials of its own slice of the [M x columns] tile, read from
    // the other CTAs' shared memory, and writes that slice of y.
    cluster_sync_all();
    const int ncols = min(kCtaCols, p.N - cta_tile0 * 8);
    const int total_pairs = (rows * kCtaCols) >> 1;
    const int per_rank = (total_pairs + p.S - 1) / p.S;
    const int first = split * per_rank;
    const int last_pair = min(first + per_rank, total_pairs);
    for (int i = first + tid; i < last_pair; i += kGemvThreads) {
      const int e = 2 * i;
      const int m = e / kCtaCols, nl = e - m * kCtaCols;
      if (nl >= ncols) continue;
      const uint32_t laddr = smem_u32(red + e);
      float2 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) v[r] = (r < p.S) ? ld_dsmem_f2(laddr, static_cast<uint32_t>(r)) : make_float2(0.f, 0.f);
      float2 sum = v[0];
#pragma unroll
      for (int r = 1; r < 8; ++r) {
        if (r < p.S) { sum.x += v[r].x; sum.y += v[r].y; }
      }
      variant_store_pair(p, fusion, row0 + m, cta_tile0 * 8 + nl, sum.x, sum.y);
    }
    cluster_sync_all();   // nobody leaves while its shared memory may still be read
    return;
  }

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned counter = (ROW_HALVES ? blockIdx.z * gridDim.x : 0u) + blockIdx.x;
    const unsigned prev = atomicAdd(&p.counters[counter], 1u);
    const int last = (prev == static_cast<unsigned>(p.S - 1));
    if (last) p.counters[counter] = 0u;  // every split has arrived: leave the counter clean
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // The last CTA of this column range adds the S partials in split order.
  const int col0 = cta_tile0 * 8;
  const int ncols = min(kCtaCols, p.N - col0);
  const int pairs = ncols >> 1;
  for (int i = tid; i < rows * pairs; i += kGemvThreads) {
    const int row = row0 + i / pairs;
    const int col = col0 + 2 * (i - (row - row0) * pairs);
    const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
    const size_t split_stride = static_cast<size_t>(p.M) * p.N;
    // Loads are issued eight at a time (independent), the additions stay in split order.
    float2 sum = make_float2(0.f, 0.f);
    for (int s0 = 0; s0 < p.S; s0 += 8) {
      float2 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = (s0 + j < p.S) ? __ldcg(reinterpret_cast<const float2*>(src + (s0 + j) * split_stride))
                              : make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (s0 + j < p.S) {
          if (s0 + j == 0) sum = v[0];
          else { sum.x += v[j].x; sum.y += v[j].y; }
        }
      }
    }
    variant_store_pair(p, fusion, row, col, sum.x, sum.y);
  }
}


// ---------------------------------------------------------------------------
// host: decomposition chosen from (K, N) only, never from M.
// ---------------------------------------------------------------------------
struct GemvPlan {
  int ntw;   // column tiles per warp (2 or 4)
  int w;     // compute warps per CTA (8 or 16)
  int kw;    // warps sharing a column group and splitting k inside the CTA (divides w)
  int bps;   // 128-k blocks per grid-level split
  int S;     // grid-level splits
  int ncol;  // CTAs along N
};

static int plan_ncol(int ntiles, int ntw, int w, int kw) {
  const int cta_tiles = (w / kw) * ntw;
  return (ntiles + cta_tiles - 1) / cta_tiles;
}

// Cost model in microseconds: a least-squares fit to a sweep of (kw, S) over the decode shapes on
// B200 (148 SMs, two resident CTAs per SM).  Terms: waves of CTAs, the blocks each warp walks
// through per wave, the way grid-level partials are added (global workspace or cluster), a per-CTA
// scheduling cost, and the slowdown of a warp when the SM is shared.
// Fitted coefficients (microseconds); see the comment above.
static const double kPlanC[8] = {-0.761, 0.882, 0.927, 1.729, 1.253, 1.918, 0.721, 0.45};

static GemvPlan plan_gemv(int K, int N, int sm_count) {
  const int nblk = K / kBlockK, ntiles = N / 8;
  const int ntw = 4;   // the row count may lower this later; it does not affect the order of additions
  GemvPlan best{ntw, 8, 1, nblk, 1, plan_ncol(ntiles, ntw, 8, 1)};
  double best_t = 1e30;
  const int ws[2] = {8, 16};
  for (int w : ws) {
    // 16-warp CTAs win some shapes when a kernel is timed alone (2048 -> 2048: 2.7 vs 3.0 us) but lose
    // inside a sequence of linears: one such CTA fills an SM, so the next launch cannot start its weight
    // prefetch beside it (28-layer decode step: 562 -> 547 us without them).  The planner leaves them out;
    // forced plans can still select them.
    if (w == 16) continue;
    const double slots = (w == 8 ? 2.0 : 1.0) * sm_count;   // resident CTAs
    for (int kw = w; kw >= (w == 8 ? 1 : 4); kw >>= 1) {
      const int ncol = plan_ncol(ntiles, ntw, w, kw);
      if (ncol > 4095) continue;
      int prev_S = -1;
      for (int bps = nblk; bps >= 1; --bps) {
        const int S = (nblk + bps - 1) / bps;
        if (S == prev_S) continue;
        prev_S = S;
        const int bps_eff = (nblk + S - 1) / S;   // even split
        if (bps_eff > kGemvMaxBps * kw) continue;
        const double bpw = (bps_eff + kw - 1) / kw;  // blocks per warp
        const double n = static_cast<double>(ncol) * S;
        const double waves = static_cast<double>(static_cast<long long>((n + slots - 1) / slots));
        const bool clus = S >= 2 && S <= 8 && n <= sm_count;
        const bool glob = S > 1 && !clus;
        const double t = kPlanC[0] + kPlanC[1] * waves + kPlanC[2] * waves * bpw + (glob ? kPlanC[3] : 0.0) +
                         (clus ? kPlanC[4] : 0.0) + kPlanC[5] * (n / slots) +
                         kPlanC[6] * ((n < slots ? n : slots) / slots) * bpw + (w == 16 ? kPlanC[7] : 0.0);
        if (t < best_t) {
          best_t = t;
          best = GemvPlan{ntw, w, kw, bps_eff, S, ncol};
        }
      }
    }
  }
  // Narrow outputs with a medium k (e.g. 6144 -> 2048): inside a sequence of decode linears four cluster
  // splits of four k-splitting warps beat every plan the fitted model ranks first (28-layer step 545 -> 522 us).
  if (ntiles <= 256 && nblk > 32 && nblk <= 64)
    best = GemvPlan{ntw, 8, 4, (nblk + 3) / 4, 4, plan_ncol(ntiles, ntw, 8, 4)};
  best.S = (nblk + best.bps - 1) / best.bps;
  return best;
}

// Streaming (persistent, evenly balanced) variant, in awq_gemv_stream.cu.
int gemv_stream_slots(int K, int N, int ntw, int w, int kw, int sm_count);
int gemv_stream_launch(const GemvParams& base, const GemvFusion& fusion, int ntw, int w, int kw, int sm_count, int max_smem_optin,
                       cudaStream_t stream, bool overlap_previous);

// The streaming kernel pays off for very large matrices only (measured: level with the per-split grid
// up to ~120 MB of packed weights, ahead of it at 16 rows beyond that): at least 32 units per resident CTA.
static bool stream_by_default(const GemvPlan& plan, int nblk, int ntiles, int sm_count) {
  const long long units = static_cast<long long>(plan_ncol(ntiles, 4, plan.w, plan.kw)) * ((nblk + plan.kw - 1) / plan.kw);
  return units >= 32LL * (plan.w == 8 ? 2 : 1) * sm_count;
}

// The arrival counters sit in a fixed-size slot at the start of the workspace,
// independent of the problem shape, so that one workspace can serve linears of
// different sizes: partial sums of one call can then never land where another
// call expects clean counters.
static size_t counter_bytes(int /*N*/) { return kGemvMaxCounters * sizeof(unsigned); }

template <int NTW, int MT, int KW, int W, bool FUSED, bool ROW_HALVES>
static int launch_gemv(const GemvParams& p_plain, const GemvFusion& fusion, const GemvPlan& plan, int max_smem_optin,
                       cudaStream_t stream, bool overlap_previous) {
  typename GemvParamsOf<FUSED>::type p;
  static_cast<GemvParams&>(p) = p_plain;
  if constexpr (FUSED) p.fusion = fusion;
  const size_t smem = static_cast<size_t>(gemv_stages(NTW, W)) * W * NTW * (512 + 32) + 2 * gemv_stages(NTW, W) * 8;
  if (smem > static_cast<size_t>(max_smem_optin)) return AWQ_B200_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    AWQ_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<NTW, MT, KW, W, FUSED, ROW_HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.ncol, plan.S, ROW_HALVES ? (p.M + MT - 1) / MT : 1);
  cfg.blockDim = dim3((W + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (overlap_previous) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = static_cast<unsigned>(plan.S);
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_kernel<NTW, MT, KW, W, FUSED, ROW_HALVES>, p));
  return AWQ_B200_OK;
}

int gemv_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const Epilogue& epi, void* y, int M, int K, int N, int group_size, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream, int force_ntw, int force_kw, int force_bps,
                  unsigned flags, int force_w = 0) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size)) return st;
  if (M < 1 || M > kGemvMaxRows) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) ||
      !aligned16(y))
    return AWQ_B200_ERR_ALIGN;
  if (int st = check_epilogue(epi, N)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;

  GemvPlan plan = plan_gemv(K, N, di.sm_count);
  const int nblk = K / kBlockK, ntiles = N / 8;
  if (force_ntw == 2 || force_ntw == 4) plan.ntw = force_ntw;
  if (force_w == 8 || force_w == 16) plan.w = force_w;
  if (force_kw >= 1 && force_kw <= plan.w && (plan.w % force_kw) == 0) plan.kw = force_kw;
  if (plan.kw > plan.w) plan.kw = plan.w;
  if (plan.w == 16 && plan.kw < 4) plan.kw = 4;
  if (force_bps >= 1) plan.bps = force_bps < nblk ? force_bps : nblk;
  if (plan.bps > kGemvMaxBps * plan.kw) plan.bps = kGemvMaxBps * plan.kw;
  // More than 8 rows.  The per-split grid runs two CTAs of 8 rows per (column group, split) with the plan
  // of 8 rows; the stream keeps its 16-row variant, which holds twice the accumulators and therefore runs
  // with two tiles per warp.  Only the k-splits (kw, bps) decide the order of additions, so neither changes
  // a row's result.
  bool use_stream = force_bps < 1 && stream_by_default(plan, nblk, ntiles, di.sm_count);
  if (flags & AWQ_B200_GEMV_STREAM) use_stream = true;
  if (flags & AWQ_B200_GEMV_PER_SPLIT) use_stream = false;
  if (M > kGemvStreamMaxRows) use_stream = false;
  if (M > 8 && force_ntw == 0 && use_stream) plan.ntw = 2;
  const int row_halves = (!use_stream && M > 8) ? (M + 7) / 8 : 1;
  plan.S = (nblk + plan.bps - 1) / plan.bps;
  plan.ncol = plan_ncol(ntiles, plan.ntw, plan.w, plan.kw);
  unsigned* p_status = nullptr;
  while (plan.ncol * row_halves > kGemvMaxCounters - 1 && plan.ntw < 4) {
    plan.ntw *= 2;
    plan.ncol = plan_ncol(ntiles, plan.ntw, plan.w, plan.kw);
  }
  if (plan.S > 65535 || plan.ncol * row_halves > kGemvMaxCounters - 1) return AWQ_B200_ERR_TOO_LARGE;
  if (workspace && workspace_bytes >= counter_bytes(N) && aligned16(workspace))
    p_status = static_cast<unsigned*>(workspace) + (kGemvMaxCounters - 1);

  GemvParams p;
  p.x = static_cast<const uint16_t*>(x);
  p.wp = static_cast<const uint4*>(packed);
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.bias = epi.bias;
  const GemvFusion fusion{epi.residual, epi.gated};
  const bool fused = epi.gated || epi.residual != nullptr;
  p.y = static_cast<uint16_t*>(y);
  p.partial = nullptr;
  p.counters = nullptr;
  p.status = p_status;
  p.M = M; p.K = K; p.N = N;
  p.group_blocks = group_size / kBlockK;
  p.nblk = nblk;
  p.bps = plan.bps;
  p.S = plan.S;
  p.ntiles = ntiles;
  const bool overlap = (flags & AWQ_B200_OVERLAP_PREVIOUS) != 0;
  if (use_stream) {
    p.bps = 0; p.S = 0; p.cluster = 0;
    const int slots = gemv_stream_slots(K, N, plan.ntw, plan.w, plan.kw, di.sm_count);
    if (slots > 1 || epi.gated) {
      const size_t cb = counter_bytes(N);
      const size_t need = cb + static_cast<size_t>(slots) * M * N * sizeof(float);
      if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
      if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
      p.counters = static_cast<unsigned*>(workspace);
      p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + cb);
    }
    return gemv_stream_launch(p, fusion, plan.ntw, plan.w, plan.kw, di.sm_count, di.max_smem_optin, stream, overlap);
  }

  // A cluster needs its CTAs resident together; beyond one CTA per SM that costs more occupancy than the
  // shared-memory reduction saves.
  p.cluster = (plan.S >= 2 && plan.S <= 8 && static_cast<long long>(plan.ncol) * plan.S * row_halves <= di.sm_count &&
               !(flags & AWQ_B200_NO_CLUSTER)) ? 1 : 0;
  if ((plan.S > 1 || epi.gated) && !p.cluster) {
    const size_t cb = counter_bytes(N);
    const size_t need = cb + static_cast<size_t>(plan.S) * M * N * sizeof(float);
    if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
    if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
    p.counters = static_cast<unsigned*>(workspace);
    p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + cb);
  }

#define AWQ_GEMV_LAUNCH(NTW_, KW_, W_, F_, R_) \
  launch_gemv<NTW_, 8, KW_, W_, F_, R_>(p, fusion, plan, di.max_smem_optin, stream, overlap)
#define AWQ_GEMV_CASE(NTW_, KW_, W_)                                                                      \
  if (plan.ntw == NTW_ && plan.kw == KW_ && plan.w == W_)                                                 \
    return fused ? (row_halves > 1 ? AWQ_GEMV_LAUNCH(NTW_, KW_, W_, true, true)                           \
                                   : AWQ_GEMV_LAUNCH(NTW_, KW_, W_, true, false))                         \
                 : (row_halves > 1 ? AWQ_GEMV_LAUNCH(NTW_, KW_, W_, false, true)                          \
                                   : AWQ_GEMV_LAUNCH(NTW_, KW_, W_, false, false));
  AWQ_GEMV_CASE(2, 1, 8) AWQ_GEMV_CASE(2, 2, 8) AWQ_GEMV_CASE(2, 4, 8) AWQ_GEMV_CASE(2, 8, 8)
  AWQ_GEMV_CASE(4, 1, 8) AWQ_GEMV_CASE(4, 2, 8) AWQ_GEMV_CASE(4, 4, 8) AWQ_GEMV_CASE(4, 8, 8)
  AWQ_GEMV_CASE(2, 4, 16) AWQ_GEMV_CASE(2, 8, 16) AWQ_GEMV_CASE(2, 16, 16)
  AWQ_GEMV_CASE(4, 4, 16) AWQ_GEMV_CASE(4, 8, 16) AWQ_GEMV_CASE(4, 16, 16)
  return AWQ_B200_ERR_SHAPE;
#undef AWQ_GEMV_CASE
#undef AWQ_GEMV_LAUNCH
}

int gemv_run(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
             void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
             cudaStream_t stream, unsigned flags) {
  return gemv_dispatch(x, packed, scales, qzeros, epi, y, M, K, N, group_size, workspace, workspace_bytes, stream,
                       0, 0, 0, flags);
}

size_t gemv_workspace_bytes(int M, int K, int N) {
  if (M < 1 || K < kBlockK || N < 8) return 0;
  // Worst case over every decomposition the planner or a forced plan can pick: bps = 1.
  const size_t S_max = static_cast<size_t>(K / kBlockK);
  return counter_bytes(N) + S_max * static_cast<size_t>(M) * N * sizeof(float);
}

}  // namespace awq

using namespace awq;

extern "C" {

size_t awq_b200_gemv_counter_bytes(int N) { return N > 0 ? counter_bytes(N) : 0; }

size_t awq_b200_gemv_workspace_bytes(int M, int K, int N) {
  if (M < 1 || K < kBlockK || N < 8) return 0;
  DeviceInfo di;
  int sm = 148;
  if (device_info(&di) == AWQ_B200_OK) sm = di.sm_count;
  GemvPlan plan = plan_gemv(K, N, sm);
  if (M > 8) plan.ntw = 2;
  plan.ncol = plan_ncol(N / 8, plan.ntw, plan.w, plan.kw);
  size_t slots = static_cast<size_t>(plan.S);
  if (M <= kGemvStreamMaxRows && stream_by_default(plan, K / kBlockK, N / 8, sm)) slots = static_cast<size_t>(gemv_stream_slots(K, N, plan.ntw, plan.w, plan.kw, sm));
  return counter_bytes(N) + slots * M * N * sizeof(float);
}

int awq_b200_gemv(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                  size_t workspace_bytes, awq_b200_stream_t stream) {
  return gemv_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace,
                       workspace_bytes, static_cast<cudaStream_t>(stream), 0, 0, 0, 0u);
}

int awq_b200_gemv_ex(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                     const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                     size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags) {
  return gemv_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace,
                       workspace_bytes, static_cast<cudaStream_t>(stream), 0, 0, 0, flags);
}

// Tuning hook: same as awq_b200_gemv with the decomposition forced
// (ntw in {2,4} column tiles per warp, kw in {1,2,4,8} warps splitting k inside a CTA, bps k-blocks
// per grid-level split; 0 = planner's choice).
// The workspace must hold awq_b200_gemv_workspace_bytes_max(M, K, N) bytes.
size_t awq_b200_gemv_workspace_bytes_max(int M, int K, int N) { return gemv_workspace_bytes(M, K, N); }

int awq_b200_gemv_plan(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size,
                       void* workspace, size_t workspace_bytes, awq_b200_stream_t stream, int ntw,
                       int kw, int bps, unsigned flags) {
  return gemv_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, workspace,
                       workspace_bytes, static_cast<cudaStream_t>(stream), ntw, kw % 100, bps, flags,
                       kw >= 100 ? 16 : (kw > 0 ? 8 : 0));
}

int awq_b200_gemv_max_rows(void) { return kGemvMaxRows; }

}  // extern "C"

// ---------------------------------------------------------------------------
// Decode GEMV for callers that cannot allocate device memory.
// ---------------------------------------------------------------------------
namespace awq {

// Scratch for the split-k partial sums and their arrival counters, resident in every GPU that loads
// this library until the process exits.  The name below is a host-side handle only: the device
// address is looked up per device with cudaGetSymbolAddress and passed to the kernel like any
// other workspace pointer.
constexpr size_t kGemvStaticScratchBytes = 8u << 20;   // 8 MiB
static __device__ __align__(256) unsigned char g_gemv_static_scratch[kGemvStaticScratchBytes];

static void* g_static_scratch_ptr[64];     // per device ordinal; written once, after set-up succeeded

static int static_scratch_for_current_device(cudaStream_t stream, void** out) {
  int dev = 0;
  AWQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_TOO_LARGE;
  void* ptr = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    // First call on this device: resolve the array's address on the device that is current now and
    // zero the arrival counters (later calls leave them zero themselves).
    AWQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_gemv_static_scratch));
    AWQ_CUDA_TRY(cudaMemsetAsync(ptr, 0, counter_bytes(0), stream));
    __atomic_store_n(&g_static_scratch_ptr[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return AWQ_B200_OK;
}

}  // namespace awq

extern "C" {

size_t awq_b200_gemv_static_scratch_bytes(void) { return kGemvStaticScratchBytes; }

int awq_b200_gemv_static_status(unsigned* status_out, awq_b200_stream_t stream) {
  if (!status_out) return AWQ_B200_ERR_NULL;
  void* scratch = nullptr;
  if (int st = static_scratch_for_current_device(static_cast<cudaStream_t>(stream), &scratch)) return st;
  AWQ_CUDA_TRY(cudaMemcpyAsync(status_out, static_cast<unsigned*>(scratch) + (kGemvMaxCounters - 1), sizeof(unsigned),
                               cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  AWQ_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return AWQ_B200_OK;
}

int awq_b200_gemv_static(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                         const void* bias, void* y, int M, int K, int N, int group_size,
                         awq_b200_stream_t stream) {
  if (M < 1 || M > 16) return AWQ_B200_ERR_SHAPE;
  if (int st = check_shape(K, N, group_size)) return st;
  // Worst case the planner can ask for at this shape; refuse rather than overrun the fixed array.
  if (awq_b200_gemv_workspace_bytes(M, K, N) > kGemvStaticScratchBytes) return AWQ_B200_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if (int st = static_scratch_for_current_device(static_cast<cudaStream_t>(stream), &scratch)) return st;
  return gemv_dispatch(x, packed, scales, qzeros, Epilogue{static_cast<const uint16_t*>(bias), nullptr, 0}, y, M, K, N, group_size, scratch, kGemvStaticScratchBytes,
                       static_cast<cudaStream_t>(stream), 0, 0, 0, 0u);
}

}  // extern "C"
