// Shared by the decode GEMV kernels: launch parameters, the tensor-core and unpack helpers, output
// stores and the cluster shared-memory primitives.
#pragma once
#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

// A CTA has W compute warps (8 or 16) plus one warp that only issues bulk copies.
constexpr int kGemvMaxBps = 32;   // per warp  // 128-k blocks per split (bounds the activation slice in smem)
constexpr int kGemvMaxRows = 16;
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

__device__ __forceinline__ float small_uint_to_float(uint32_t v) {   // exact for v < 2^23, no I2F
  return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

__device__ __forceinline__ void store_out1(uint16_t* y, const uint16_t* bias, size_t row_off, int col, float a) {
  __half h = __float2half_rn(a);
  if (bias != nullptr) h = __hadd(h, __ushort_as_half(bias[col]));
  y[row_off + col] = __half_as_ushort(h);
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
