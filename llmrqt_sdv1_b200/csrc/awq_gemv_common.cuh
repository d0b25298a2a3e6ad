// Shared by the decode GEMV kernels: launch parameters, the tensor-core and unpack helpers, output
// stores and the cluster shared-memory primitives.
#pragma once
#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

// A CTA has W compute warps (8 or 16) plus one warp that only issues bulk copies.
constexpr int kGemvMaxBps = 32;   // per warp  // 128-k blocks per split (bounds the activation slice in smem)
constexpr int kGemvMaxRows = 64;          // 8 rows per CTA; more rows = more CTAs per (column group, split)
constexpr int kGemvStreamMaxRows = 16;    // the persistent stream form holds at most 16 rows per CTA
// Arrival counters at the start of the workspace (fixed size; the last slot is the status word).
constexpr int kGemvMaxCounters = 4096;
// 128-k blocks in flight per CTA (bulk copies): 5 x 17 KiB or 6 x 8.5 KiB of shared memory.
__host__ __device__ constexpr int gemv_stages(int ntw, int w) { return w == 16 ? (ntw == 4 ? 3 : 4) : (ntw == 4 ? 5 : 6); }

struct GemvParams {
  const uint16_t* x;
  const uint4* wp;
  const uint16_t* scales;
  const uint32_t* qzeros;
  const uint16_t* bias;
  uint16_t* y;
  float* partial;
  unsigned* counters;
  unsigned* status;    // last counter slot: 0, or the code of a device-side wait that expired
  int M, K, N;
  int group_blocks;  // group_size / 128
  int nblk;          // K / 128
  int bps;           // blocks per split
  int S;             // number of splits
  int ntiles;        // N / 8
  int cluster;       // 1: the S splits of a column range form one thread-block cluster and reduce over DSMEM
};
// What a FUSED kernel variant carries besides the bias (see struct Epilogue).  The unfused variants keep
// the plain parameter block, so their code does not change with what the fused ones can do.
struct GemvFusion {
  const uint16_t* residual;
  int gated;
};
struct GemvParamsFused : GemvParams {
  GemvFusion fusion;
};
template <bool FUSED> struct GemvParamsOf { using type = GemvParams; };
template <> struct GemvParamsOf<true> { using type = GemvParamsFused; };

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

// One packed word (8 nibbles) -> four half2 for the tensor core, without scaling and without
// removing the constant that carries the nibble into an fp16 mantissa:
// out[0], out[2] hold 1024 + q (nibbles 0/4 and 2/6 or-ed into the mantissa of 2^10);
// out[1], out[3] hold 64 + q (nibbles 1/5 and 3/7 or-ed into the mantissa of 2^6).
// The constants are removed afterwards through the per-block activation sums (kCodeOffsetLo/Hi
// are the matching A-operand rows of that sum).  Five logic operations per word.
constexpr uint32_t kCodeOffsetLo = 0x64006400u;   // 1024.0 x2
constexpr uint32_t kCodeOffsetHi = 0x54005400u;   // 64.0 x2
__device__ __forceinline__ void unpack_codes(uint32_t w, uint32_t out[4]) {
  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u;
  const uint32_t w8 = w >> 8;
  out[0] = lop3_and_or(w, kLoMask, kCodeOffsetLo);
  out[1] = lop3_and_or(w, kHiMask, kCodeOffsetHi);
  out[2] = lop3_and_or(w8, kLoMask, kCodeOffsetLo);
  out[3] = lop3_and_or(w8, kHiMask, kCodeOffsetHi);
}

// D = A * B with a zero C operand (no accumulator registers to clear beforehand).
__device__ __forceinline__ void mma_16816_first(float acc[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(acc[0]), "=f"(acc[1]), "=f"(acc[2]), "=f"(acc[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// The arithmetic of one 128-k block of one warp, shared by the decode kernels.  Lane (g, c) holds, per row
// half mh, the activations of row 8*mh + g at k = 32c .. 32c+31 (xv), and per column tile t the four packed
// words 4c .. 4c+3 of column 8t + g (wv).
//
// gemv_block_sums: per-block activation sums from the tensor core.  A rows 0..7 are all ones (-> S[m] =
// sum_k x[m,k]), rows 8..15 hold the constant carried by the code at that k, 1024 or 64 (-> H[m]).  Two short
// chains; T[mh] = (S[2c], S[2c+1], H[2c], H[2c+1]) of rows 8*mh + 2c, +1.
template <int MH>
__device__ __forceinline__ void gemv_block_sums(const uint4 (&xv)[MH][4], float4 (&T)[MH]) {
#pragma unroll
  for (int mh = 0; mh < MH; ++mh) {
    float SH0[4], SH1[4];
    constexpr uint32_t kOne = 0x3C003C00u;
    mma_16816_first(SH0, kOne, kCodeOffsetLo, kOne, kCodeOffsetHi, xv[mh][0].x, xv[mh][0].y);
    mma_16816_first(SH1, kOne, kCodeOffsetLo, kOne, kCodeOffsetHi, xv[mh][0].z, xv[mh][0].w);
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      mma_16816(SH0, kOne, kCodeOffsetLo, kOne, kCodeOffsetHi, xv[mh][i].x, xv[mh][i].y);
      mma_16816(SH1, kOne, kCodeOffsetLo, kOne, kCodeOffsetHi, xv[mh][i].z, xv[mh][i].w);
    }
    T[mh] = make_float4(SH0[0] + SH1[0], SH0[1] + SH1[1], SH0[2] + SH1[2], SH0[3] + SH1[3]);
  }
}

// gemv_block_pairs: for each pair of column tiles (the 16 rows of the mma A operand),
//   acc += s * ( sum_k x * code - H - z * S )
// with two independent accumulation chains per block, both starting from zero.  acc[mh][q] holds rows
// 8*mh + 2c, +1 of columns g (elements 0, 1) and 8 + g (elements 2, 3) of pair q.
template <int NTW, int MH>
__device__ __forceinline__ void gemv_block_pairs(const uint4 (&wv)[NTW], const float (&sc)[NTW], const float (&zp)[NTW],
                                                 const uint4 (&xv)[MH][4], const float4 (&T)[MH],
                                                 float (&acc)[MH][NTW / 2][4]) {
#pragma unroll
  for (int q = 0; q < NTW / 2; ++q) {
    const uint32_t wa[4] = {wv[2 * q].x, wv[2 * q].y, wv[2 * q].z, wv[2 * q].w};
    const uint32_t wb[4] = {wv[2 * q + 1].x, wv[2 * q + 1].y, wv[2 * q + 1].z, wv[2 * q + 1].w};
    const float sa = sc[2 * q], za = zp[2 * q], sb = sc[2 * q + 1], zb = zp[2 * q + 1];
    float blk[MH][2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t qa[4], qb[4];
      unpack_codes(wa[i], qa);
      unpack_codes(wb[i], qb);
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) {
        if (i == 0) {
          mma_16816_first(blk[mh][0], qa[0], qb[0], qa[1], qb[1], xv[mh][i].x, xv[mh][i].y);
          mma_16816_first(blk[mh][1], qa[2], qb[2], qa[3], qb[3], xv[mh][i].z, xv[mh][i].w);
        } else {
          mma_16816(blk[mh][0], qa[0], qb[0], qa[1], qb[1], xv[mh][i].x, xv[mh][i].y);
          mma_16816(blk[mh][1], qa[2], qb[2], qa[3], qb[3], xv[mh][i].z, xv[mh][i].w);
        }
      }
    }
#pragma unroll
    for (int mh = 0; mh < MH; ++mh) {
      // sum_k x*code = chain0 + chain1 - H   (H removes the constants 1024 / 64 carried by the codes)
      const float d0 = (blk[mh][0][0] + blk[mh][1][0]) - T[mh].z, d1 = (blk[mh][0][1] + blk[mh][1][1]) - T[mh].w;
      const float d2 = (blk[mh][0][2] + blk[mh][1][2]) - T[mh].z, d3 = (blk[mh][0][3] + blk[mh][1][3]) - T[mh].w;
      acc[mh][q][0] = fmaf(sa, fmaf(-za, T[mh].x, d0), acc[mh][q][0]);
      acc[mh][q][1] = fmaf(sa, fmaf(-za, T[mh].y, d1), acc[mh][q][1]);
      acc[mh][q][2] = fmaf(sb, fmaf(-zb, T[mh].x, d2), acc[mh][q][2]);
      acc[mh][q][3] = fmaf(sb, fmaf(-zb, T[mh].y, d3), acc[mh][q][3]);
    }
  }
}

__device__ __forceinline__ float small_uint_to_float(uint32_t v) {   // exact for v < 2^23, no I2F
  return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

// The stores of a kernel variant: FUSED = false is the bias-only epilogue, FUSED = true the full one.
// y = fp16(acc) then, with a bias, fp16(y + bias): the two roundings of the reference's `out + bias` on an
// fp16 tensor.
__device__ __forceinline__ void store_out2(uint16_t* y, const uint16_t* bias, size_t row_off, int col,
                                           float a, float b) {
  uint32_t v = pack_half2(a, b);
  if (bias != nullptr) {
    const uint32_t bv = *reinterpret_cast<const uint32_t*>(bias + col);
    asm("add.f16x2 %0, %1, %2;" : "=r"(v) : "r"(v), "r"(bv));
  }
  *reinterpret_cast<uint32_t*>(y + row_off + col) = v;
}
__device__ __forceinline__ void store_out1(uint16_t* y, const uint16_t* bias, size_t row_off, int col, float a) {
  __half h = __float2half_rn(a);
  if (bias != nullptr) h = __hadd(h, __ushort_as_half(bias[col]));
  y[row_off + col] = __half_as_ushort(h);
}
// The stores of a kernel variant: P = GemvParams is the bias-only epilogue, P = GemvParamsFused the full one
// (`f` is its fusion block; ignored otherwise).
__device__ __forceinline__ void variant_store_one(const GemvParams& p, const GemvFusion* f, int m, int col, float a) {
  if (f != nullptr) epilogue_store_one(p.y, Epilogue{p.bias, f->residual, f->gated}, m, p.N, col, a);
  else store_out1(p.y, p.bias, static_cast<size_t>(m) * p.N, col, a);
}
__device__ __forceinline__ void variant_store_pair(const GemvParams& p, const GemvFusion* f, int m, int col, float a,
                                                   float b) {
  if (f != nullptr) epilogue_store_pair(p.y, Epilogue{p.bias, f->residual, f->gated}, m, p.N, col, a, b);
  else store_out2(p.y, p.bias, static_cast<size_t>(m) * p.N, col, a, b);
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float2 ld_dsmem_f2(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
  return v;
}

}  // namespace awq
