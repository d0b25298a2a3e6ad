// tcgen05 / TMEM / tiled-TMA PTX wrappers and the host-side tensor-map encoder lookup, shared by
// the tensor-core kernels.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace awq {

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of
// 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address
  d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                    // stride byte offset: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;                            // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                            // SWIZZLE_128B
  return d;
}


// A operand taken from tensor memory (lane = row, two 16-bit elements per 32-bit column), B from shared memory.
__device__ __forceinline__ void tcgen05_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Whole-warp forms: every lane of a converged warp executes the call with the same operands and one
// elected lane issues.  Keeping the issuing loop warp-uniform lets the operands live in uniform
// registers, which is what makes the per-instruction issue cost small.
__device__ __forceinline__ void tcgen05_mma_f16_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Eight k-steps (128 k) of A-from-tensor-memory MMAs into one accumulator, then two commits, all
// issued by one elected lane under a single election: A advances 8 tensor-memory columns per step;
// the B descriptor advances `step_lo` (in 16-byte units) per step inside a 64-k half and `half_lo`
// between the two halves.  `accumulate_first` = 0 starts a new accumulation.  Keeping the whole
// group in one statement keeps the issuing warp's instruction count per unit small, which matters
// because it shares its scheduler with busy dequant warps.
__device__ __forceinline__ void tcgen05_mma_f16_ts_k8_commit2_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                                   uint32_t step_lo, uint32_t half_lo, uint32_t idesc,
                                                                   uint32_t accumulate_first, uint32_t bar0,
                                                                   uint32_t bar1) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b32 a, lo, hi, lo0;\n\t.reg .b64 d;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "mov.b64 {lo0, hi}, %2;\n\t"
      // first half: steps 0..3
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %5, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 a, %1, 8;\n\t  add.u32 lo, lo0, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      // second half: steps 4..7
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo0, %4;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "add.u32 a, a, 8;\n\t  add.u32 lo, lo, %3;\n\t  mov.b64 d, {lo, hi};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %5, p;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%8];\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(step_lo), "r"(half_lo), "r"(idesc), "r"(accumulate_first),
        "r"(bar0), "r"(bar1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_warp(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Order in which a persistent grid walks the (row tile, column tile) grid: bands of kTileBandRows row
// tiles, and inside a band row tiles fastest.  The ~148 tiles in flight then cover a compact block
// (8 row tiles x ~18 column tiles) instead of every row tile of a few column tiles, so the working
// set of one wave (activations + packed weights) stays small enough to be re-read from L2.
constexpr int kTileBandRows = 8;
__device__ __forceinline__ void tile_coords(int tile, int mtiles, int ntiles, int* mi, int* ni) {
  const int band_tiles = kTileBandRows * ntiles;
  const int band = tile / band_tiles;
  const int first = band * kTileBandRows;
  const int rows = min(kTileBandRows, mtiles - first);
  const int r = tile - band * band_tiles;
  *ni = r / rows;
  *mi = first + (r - *ni * rows);
}

// Instruction descriptor for kind::f16: D fp32, A and B fp16, both K-major, given M and N.
__host__ __device__ constexpr uint32_t make_f16_idesc(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// cuTensorMapEncodeTiled, looked up once through the runtime (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int get_encode(EncodeTiledFn* out);

}  // namespace awq
