// Decode path: split-K W4A16 GEMV for 1 <= M <= 16 rows.
//
// One pass over the packed weights serves all rows.  Work unit = one 128-k
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
#include "awq_common.cuh"

namespace awq {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;
constexpr int kGemvMaxBps = 16;   // 128-k blocks per split (bounds the activation slice in smem)
constexpr int kGemvMaxRows = 16;
constexpr int kGemvUnitsInFlight = 8;  // 128-bit weight loads in flight per thread

struct GemvParams {
  const uint16_t* x;
  const uint4* wp;
  const uint16_t* scales;
  const uint32_t* qzeros;
  const uint16_t* bias;
  uint16_t* y;
  float* partial;
  unsigned* counters;
  int M, K, N;
  int group_blocks;  // group_size / 128
  int nblk;          // K / 128
  int bps;           // blocks per split
  int S;             // number of splits
  int ntiles;        // N / 8
};

__device__ __forceinline__ void mma_16816(float acc[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// y = fp16(acc) then, with a bias, fp16(y + bias): the two roundings of the
// reference's `out + bias` on an fp16 tensor.
__device__ __forceinline__ void store_out2(uint16_t* y, const uint16_t* bias, size_t row_off, int col,
                                           float a, float b) {
  uint32_t v = pack_half2(a, b);
  if (bias != nullptr) {
    const uint32_t bv = *reinterpret_cast<const uint32_t*>(bias + col);
    asm("add.f16x2 %0, %1, %2;" : "=r"(v) : "r"(v), "r"(bv));
  }
  *reinterpret_cast<uint32_t*>(y + row_off + col) = v;
}

// One packed word (8 nibbles) -> four half2 for the tensor core, without scaling:
// out[0], out[2] hold the exact codes q (nibbles 0/4 and 2/6: (q | 0x6400) - 1024);
// out[1], out[3] hold 64 + q (nibbles 1/5 and 3/7 or-ed into the mantissa of 2^6),
// whose constant 64 is removed afterwards through the per-block activation sums.
__device__ __forceinline__ void unpack_codes(uint32_t w, uint32_t out[4]) {
  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u;
  constexpr uint32_t k1024 = 0x64006400u, k64 = 0x54005400u;
  const uint32_t w8 = w >> 8;
  out[0] = h2_sub(lop3_and_or(w, kLoMask, k1024), k1024);
  out[1] = lop3_and_or(w, kHiMask, k64);
  out[2] = h2_sub(lop3_and_or(w8, kLoMask, k1024), k1024);
  out[3] = lop3_and_or(w8, kHiMask, k64);
}

__device__ __forceinline__ float small_uint_to_float(uint32_t v) {   // exact for v < 2^23, no I2F
  return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

// NTW (2 or 4) column tiles per warp, handled as NTW/2 pairs of 16 columns; MT = 8 or 16 rows.
//
// Arithmetic per 128-k block b, column n, row m (all fp32 after the tensor core):
//   y[m,n] += s[b,n] * ( sum_k x[m,k] * code[k,n]  -  z[b,n] * sum_k x[m,k] )
// The 16 columns of a pair are the rows of the mma A operand (the weights), the
// activations are the B operand (8 rows of x per mma), so one m16n8k16 covers
// 16 columns x 16 k.  The two activation sums per block and row (all k, and 64x
// the k fed as "64 + q") come from the tensor core as well, once per CTA.
__device__ __forceinline__ void store_out1(uint16_t* y, const uint16_t* bias, size_t row_off, int col, float a) {
  __half h = __float2half_rn(a);
  if (bias != nullptr) h = __hadd(h, __ushort_as_half(bias[col]));
  y[row_off + col] = __half_as_ushort(h);
}

template <int NTW, int MT>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_kernel(const GemvParams p) {
  static_assert(NTW == 2 || NTW == 4, "column tiles are processed in pairs");
  constexpr int NP = NTW / 2;    // pairs per warp
  constexpr int MH = MT / 8;     // row halves
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_last;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = blockIdx.y;
  const int b0 = split * p.bps;
  const int nb = min(p.bps, p.nblk - b0);
  const int row_stride = p.bps * 256 + 64;  // bytes; +64 keeps rows g and g+1 on disjoint banks
  unsigned char* tsm = smem + MT * row_stride;   // [bps][MH][4 lanes c] x float4 {S(2c), S(2c+1), H(2c), H(2c+1)}
  unsigned char* szsm = tsm + p.bps * MH * 64;   // [bps][8 * NTW tiles][8 columns] x float2 {scale, zero}

  const int tile0 = (blockIdx.x * kGemvWarps + warp) * NTW;
  int tile[NTW];
#pragma unroll
  for (int t = 0; t < NTW; ++t) tile[t] = min(tile0 + t, p.ntiles - 1);  // clamp: loads stay in range

  const size_t block_stride_u4 = static_cast<size_t>(p.N) * 4;  // uint4 per 128-k block
  const int zcols = p.N >> 3;

  // Register ring of D = NTW * PB 128-bit weight loads: PB k-blocks are in flight
  // per thread at all times.  One base pointer per tile; the block offset is a
  // widening multiply-add.
  constexpr int PB = kGemvUnitsInFlight / NTW;
  constexpr int D = NTW * PB;
  uint4 wr[D];
  const uint4* wbase[NTW];
#pragma unroll
  for (int t = 0; t < NTW; ++t)
    wbase[t] = p.wp + static_cast<size_t>(b0) * block_stride_u4 + static_cast<size_t>(tile[t]) * 32 + lane;
  const unsigned block_stride32 = static_cast<unsigned>(p.N) * 4u;
  auto issue_load = [&](int bl, int t, uint4& w) {
    w = ldg_stream(wbase[t] + static_cast<unsigned long long>(static_cast<unsigned>(bl)) * block_stride32);
  };
#pragma unroll
  for (int j = 0; j < D; ++j) {
    if (j / NTW < nb) issue_load(j / NTW, j % NTW, wr[j]);
  }

  // Scale and zero point of every (block, column) of this CTA go to shared memory
  // once, already as fp32 pairs {s, z}; the main loop then needs no global loads
  // besides the weights.  One item = 8 columns (one qzeros word, 8 scales).
  {
    constexpr int kCtaTiles = kGemvWarps * NTW;
    const int cta_tile0 = blockIdx.x * kCtaTiles;
    for (int i = tid; i < nb * kCtaTiles; i += kGemvThreads) {
      const int bl = i / kCtaTiles, tt = i - bl * kCtaTiles;
      const int tl = min(cta_tile0 + tt, p.ntiles - 1);
      const int grp = (b0 + bl) / p.group_blocks;
      const uint32_t zw = __ldg(p.qzeros + static_cast<size_t>(grp) * zcols + tl);
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(p.scales + static_cast<size_t>(grp) * p.N + tl * 8));
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
      float4* dst = reinterpret_cast<float4*>(szsm + (static_cast<size_t>(bl) * kCtaTiles + tt) * 64);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float s0 = __half2float(__ushort_as_half(static_cast<unsigned short>(sw[h] & 0xFFFFu)));
        const float s1 = __half2float(__ushort_as_half(static_cast<unsigned short>(sw[h] >> 16)));
        const float z0 = small_uint_to_float((zw >> awq_slot_shift(2 * h)) & 0xFu);
        const float z1 = small_uint_to_float((zw >> awq_slot_shift(2 * h + 1)) & 0xFu);
        dst[h] = make_float4(s0, z0, s1, z1);
      }
    }
  }

  // Stage this split's activation slice.  Chunk j (8 halves) of a block lands at
  // slot (j % 4) * 4 + j / 4 so that lane c's i-th 128-bit read (chunk 4c + i)
  // is conflict free.
  {
    const int chunks_per_row = nb * 16;
    const int total = MT * chunks_per_row;
    for (int i = tid; i < total; i += kGemvThreads) {
      const int r = i / chunks_per_row;
      const int cj = i - r * chunks_per_row;
      const int bl = cj >> 4, j = cj & 15;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < p.M)
        v = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(r) * p.K +
                                                 static_cast<size_t>(b0 + bl) * kBlockK + j * 8));
      const int slot = (j & 3) * 4 + (j >> 2);
      *reinterpret_cast<uint4*>(smem + r * row_stride + bl * 256 + slot * 16) = v;
    }
  }
  __syncthreads();

  const unsigned char* xrow = smem + g * row_stride + c * 16;

  // Per-block activation sums, through the tensor core: S[m] = sum_k x[m,k] and
  // H[m] = 64 * sum over the k that are fed as (64 + q).
  for (int bl = warp; bl < nb; bl += kGemvWarps) {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh) {
      float S[4] = {0.f, 0.f, 0.f, 0.f}, H[4] = {0.f, 0.f, 0.f, 0.f};
      constexpr uint32_t kOne = 0x3C003C00u, k64 = 0x54005400u;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xrow + mh * 8 * row_stride + bl * 256 + i * 64);
        mma_16816(S, kOne, kOne, kOne, kOne, xv.x, xv.y);
        mma_16816(S, kOne, kOne, kOne, kOne, xv.z, xv.w);
        mma_16816(H, 0u, 0u, k64, k64, xv.x, xv.y);
        mma_16816(H, 0u, 0u, k64, k64, xv.z, xv.w);
      }
      if (g == 0)
        *reinterpret_cast<float4*>(tsm + ((bl * MH + mh) * 4 + c) * 16) = make_float4(S[0], S[1], H[0], H[1]);
    }
  }
  __syncthreads();

  float acc[MH][NP][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int q = 0; q < NP; ++q) acc[mh][q][0] = acc[mh][q][1] = acc[mh][q][2] = acc[mh][q][3] = 0.f;

  for (int bl0 = 0; bl0 < nb; bl0 += PB) {
#pragma unroll
    for (int pb = 0; pb < PB; ++pb) {
      const int bl = bl0 + pb;
      if (bl < nb) {
        uint4 xv[MH][4];
        float4 T[MH];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            xv[mh][i] = *reinterpret_cast<const uint4*>(xrow + mh * 8 * row_stride + bl * 256 + i * 64);
          T[mh] = *reinterpret_cast<const float4*>(tsm + ((bl * MH + mh) * 4 + c) * 16);
        }
#pragma unroll
        for (int q = 0; q < NP; ++q) {
          const int ja = pb * NTW + 2 * q, jb = ja + 1;
          const uint32_t wa[4] = {wr[ja].x, wr[ja].y, wr[ja].z, wr[ja].w};
          const uint32_t wb[4] = {wr[jb].x, wr[jb].y, wr[jb].z, wr[jb].w};
          const float2* szp = reinterpret_cast<const float2*>(
              szsm + ((static_cast<size_t>(bl) * (kGemvWarps * NTW) + warp * NTW + 2 * q) * 8 + g) * 8);
          const float2 sza = szp[0], szb = szp[8];
          const float sa = sza.x, za = sza.y, sb = szb.x, zb = szb.y;
          if (bl + PB < nb) {   // refill the two slots just read
            issue_load(bl + PB, 2 * q, wr[ja]);
            issue_load(bl + PB, 2 * q + 1, wr[jb]);
          }
          float blk[MH][4];
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {   // start from -H so the "+64" terms cancel inside the chain
            blk[mh][0] = -T[mh].z; blk[mh][1] = -T[mh].w; blk[mh][2] = -T[mh].z; blk[mh][3] = -T[mh].w;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t qa[4], qb[4];
            unpack_codes(wa[i], qa);
            unpack_codes(wb[i], qb);
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
              mma_16816(blk[mh], qa[0], qb[0], qa[1], qb[1], xv[mh][i].x, xv[mh][i].y);
              mma_16816(blk[mh], qa[2], qb[2], qa[3], qb[3], xv[mh][i].z, xv[mh][i].w);
            }
          }
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            acc[mh][q][0] = fmaf(sa, fmaf(-za, T[mh].x, blk[mh][0]), acc[mh][q][0]);
            acc[mh][q][1] = fmaf(sa, fmaf(-za, T[mh].y, blk[mh][1]), acc[mh][q][1]);
            acc[mh][q][2] = fmaf(sb, fmaf(-zb, T[mh].x, blk[mh][2]), acc[mh][q][2]);
            acc[mh][q][3] = fmaf(sb, fmaf(-zb, T[mh].y, blk[mh][3]), acc[mh][q][3]);
          }
        }
      }
    }
  }

  // ---- epilogue: this thread holds rows m = 8*mh + 2c, +1 of columns n and n + 8 ------------
  const bool direct = (p.S == 1);
#pragma unroll
  for (int q = 0; q < NP; ++q) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (tile0 + 2 * q + half >= p.ntiles) continue;
      const int n = (tile0 + 2 * q + half) * 8 + g;
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int m = mh * 8 + 2 * c + e;
          if (m >= p.M) continue;
          const float v = acc[mh][q][half * 2 + e];
          if (direct) store_out1(p.y, p.bias, static_cast<size_t>(m) * p.N, n, v);
          else __stcg(p.partial + (static_cast<size_t>(split) * p.M + m) * p.N + n, v);
        }
      }
    }
  }
  if (direct) return;

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&p.counters[blockIdx.x], 1u);
    const int last = (prev == static_cast<unsigned>(p.S - 1));
    if (last) p.counters[blockIdx.x] = 0u;  // every split has arrived: leave the counter clean
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // The last CTA of this column range adds the S partials in split order.
  const int col0 = blockIdx.x * (kGemvWarps * NTW * 8);
  const int ncols = min(kGemvWarps * NTW * 8, p.N - col0);
  const int pairs = ncols >> 1;
  for (int i = tid; i < p.M * pairs; i += kGemvThreads) {
    const int row = i / pairs;
    const int col = col0 + 2 * (i - row * pairs);
    const float* src = p.partial + static_cast<size_t>(row) * p.N + col;
    const size_t split_stride = static_cast<size_t>(p.M) * p.N;
    float2 sum = __ldcg(reinterpret_cast<const float2*>(src));
    for (int s = 1; s < p.S; ++s) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(src + s * split_stride));
      sum.x += v.x;
      sum.y += v.y;
    }
    store_out2(p.y, p.bias, static_cast<size_t>(row) * p.N, col, sum.x, sum.y);
  }
}

// ---------------------------------------------------------------------------
// host: decomposition chosen from (K, N) only, never from M.
// ---------------------------------------------------------------------------
struct GemvPlan {
  int ntw;
  int bps;
  int S;
  int ncol;
};

static GemvPlan plan_gemv(int K, int N, int sm_count) {
  const int nblk = K / kBlockK, ntiles = N / 8;
  const int slots = sm_count * 2;
  // Cost model in microseconds: a CTA streams bps*ntw units of 4 KiB; two CTAs
  // share one SM's slice of HBM bandwidth (~44 KB/us).
  const double t_fix = 1.2, t_unit = 0.19, t_red = 0.4, t_red_split = 0.04;
  GemvPlan best{2, 1, nblk, 0};
  double best_t = 1e30;
  const int ntws[2] = {4, 2};
  for (int ntw : ntws) {
    const int ncol = (ntiles + kGemvWarps * ntw - 1) / (kGemvWarps * ntw);
    int prev_S = -1;
    for (int bps = kGemvMaxBps; bps >= 1; --bps) {
      const int S = (nblk + bps - 1) / bps;
      if (S == prev_S) continue;
      prev_S = S;
      const int bps_eff = (nblk + S - 1) / S;  // even split
      const long long nctas = static_cast<long long>(ncol) * S;
      const long long waves = (nctas + slots - 1) / slots;
      double t = waves * (t_fix + bps_eff * ntw * t_unit);
      if (S > 1) t += t_red + S * t_red_split;
      if (t < best_t) {
        best_t = t;
        best = GemvPlan{ntw, bps_eff, S, ncol};
      }
    }
  }
  best.S = (nblk + best.bps - 1) / best.bps;
  return best;
}

// The arrival counters sit in a fixed-size slot at the start of the workspace,
// independent of the problem shape, so that one workspace can serve linears of
// different sizes: partial sums of one call can then never land where another
// call expects clean counters.
constexpr int kGemvMaxCounters = 4096;
static size_t counter_bytes(int /*N*/) { return kGemvMaxCounters * sizeof(unsigned); }

template <int NTW, int MT>
static int launch_gemv(const GemvParams& p, const GemvPlan& plan, int max_smem_optin, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(MT) * (p.bps * 256 + 64) + static_cast<size_t>(p.bps) * (MT / 8) * 64 +
                      static_cast<size_t>(p.bps) * kGemvWarps * NTW * 64;
  if (smem > static_cast<size_t>(max_smem_optin)) return AWQ_B200_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    AWQ_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<NTW, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  }
  dim3 grid(plan.ncol, plan.S);
  gemv_kernel<NTW, MT><<<grid, kGemvThreads, smem, stream>>>(p);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

int gemv_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream, int force_ntw, int force_bps) {
  if (!x || !packed || !scales || !qzeros || !y) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size)) return st;
  if (M < 1 || M > kGemvMaxRows) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(packed) || !aligned16(scales) || !aligned16(qzeros) ||
      !aligned16(y) || (bias && !aligned16(bias)))
    return AWQ_B200_ERR_ALIGN;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  if (di.cc_major != 10) return AWQ_B200_ERR_ARCH;

  GemvPlan plan = plan_gemv(K, N, di.sm_count);
  if (force_ntw == 2 || force_ntw == 4) plan.ntw = force_ntw;
  if (force_bps >= 1 && force_bps <= kGemvMaxBps) plan.bps = force_bps;
  // The 16-row variant keeps twice the accumulators: run it with two tiles per warp.  Only the
  // k-split decides the order of additions, so this cannot change a row's result.
  if (M > 8 && force_ntw == 0) plan.ntw = 2;
  const int nblk = K / kBlockK, ntiles = N / 8;
  plan.S = (nblk + plan.bps - 1) / plan.bps;
  plan.ncol = (ntiles + kGemvWarps * plan.ntw - 1) / (kGemvWarps * plan.ntw);
  while (plan.ncol > kGemvMaxCounters && plan.ntw < 4) {
    plan.ntw *= 2;
    plan.ncol = (ntiles + kGemvWarps * plan.ntw - 1) / (kGemvWarps * plan.ntw);
  }
  if (plan.S > 65535 || plan.ncol > kGemvMaxCounters) return AWQ_B200_ERR_TOO_LARGE;

  GemvParams p;
  p.x = static_cast<const uint16_t*>(x);
  p.wp = static_cast<const uint4*>(packed);
  p.scales = static_cast<const uint16_t*>(scales);
  p.qzeros = reinterpret_cast<const uint32_t*>(qzeros);
  p.bias = static_cast<const uint16_t*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.partial = nullptr;
  p.counters = nullptr;
  p.M = M; p.K = K; p.N = N;
  p.group_blocks = group_size / kBlockK;
  p.nblk = nblk;
  p.bps = plan.bps;
  p.S = plan.S;
  p.ntiles = ntiles;
  if (plan.S > 1) {
    const size_t cb = counter_bytes(N);
    const size_t need = cb + static_cast<size_t>(plan.S) * M * N * sizeof(float);
    if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
    if (!aligned16(workspace)) return AWQ_B200_ERR_ALIGN;
    p.counters = static_cast<unsigned*>(workspace);
    p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + cb);
  }

  const bool wide = M > 8;
#define AWQ_GEMV_CASE(NTW_)                                                                  \
  case NTW_:                                                                                 \
    return wide ? launch_gemv<NTW_, 16>(p, plan, di.max_smem_optin, stream)                  \
                : launch_gemv<NTW_, 8>(p, plan, di.max_smem_optin, stream);
  switch (plan.ntw) {
    AWQ_GEMV_CASE(2)
    AWQ_GEMV_CASE(4)
    default: return AWQ_B200_ERR_SHAPE;
  }
#undef AWQ_GEMV_CASE
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
  const GemvPlan plan = plan_gemv(K, N, sm);
  return counter_bytes(N) + static_cast<size_t>(plan.S) * M * N * sizeof(float);
}

int awq_b200_gemv(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                  size_t workspace_bytes, awq_b200_stream_t stream) {
  return gemv_dispatch(x, packed, scales, qzeros, bias, y, M, K, N, group_size, workspace,
                       workspace_bytes, static_cast<cudaStream_t>(stream), 0, 0);
}

// Tuning hook: same as awq_b200_gemv with the decomposition forced
// (ntw in {2,4} column tiles per warp, bps in 1..16 k-blocks per split; 0 = planner's choice).
// The workspace must hold awq_b200_gemv_workspace_bytes_max(M, K, N) bytes.
size_t awq_b200_gemv_workspace_bytes_max(int M, int K, int N) { return gemv_workspace_bytes(M, K, N); }

int awq_b200_gemv_plan(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size,
                       void* workspace, size_t workspace_bytes, awq_b200_stream_t stream, int ntw,
                       int bps) {
  return gemv_dispatch(x, packed, scales, qzeros, bias, y, M, K, N, group_size, workspace,
                       workspace_bytes, static_cast<cudaStream_t>(stream), ntw, bps);
}

int awq_b200_gemv_max_rows(void) { return kGemvMaxRows; }

}  // extern "C"
