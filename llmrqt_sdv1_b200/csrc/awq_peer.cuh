// Flag-array layout, wire format and limits of the one-shot peer exchange (awq_allreduce.cu), shared with the
// decode kernel whose epilogue performs the push form of the exchange itself (awq_decode_i8.cu).
#pragma once
#include "awq_common.cuh"

namespace awq {

constexpr int kArMaxWorld = 16;
constexpr unsigned long long kArWaitLimitCycles = 4000000000ull;   // default limit of a wait on a peer: ~2 s at 2 GHz

// Flag array layout (uint32 words) in each rank's symmetric flag buffer:
//   [0, 16)   ready[r]   written by rank r
//   [16, 32)  done[r]    written by rank r
//   [32]      epoch of the last completed call (local)
//   [33]      blocks of the current call that finished summing (local)
//   [34]      status: 0, or 1 / 2 when the ready / done wait expired, 3 for the push variant's wait (local, sticky)
//   [35], [36] epoch and finished-block counter of the push variant (local)
//   [37]      limit of a wait on a peer in units of 1024 SM cycles; 0 = the default of ~2 s (local, set by the host)
constexpr int kArReadyOff = 0, kArDoneOff = 16, kArEpochOff = 32, kArBlocksOff = 33, kArStatusOff = 34;
constexpr int kArPushEpochOff = 35, kArPushBlocksOff = 36, kArLimitOff = 37;
static_assert(kArStatusOff == AWQ_B200_PEER_STATUS_WORD && kArLimitOff == AWQ_B200_PEER_WAIT_LIMIT_WORD,
              "the header documents these two words");
constexpr int kArMaxBlocks = 64;
constexpr int kArFlagWords = 64;

__device__ __forceinline__ unsigned long long wait_limit_cycles(const unsigned* my_flags) {
  const unsigned kcycles = my_flags[kArLimitOff];
  return kcycles != 0u ? static_cast<unsigned long long>(kcycles) << 10 : kArWaitLimitCycles;
}

__device__ __forceinline__ void st_wire_16(void* p, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
               : "memory");
}
__device__ __forceinline__ uint4 ld_wire_16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// One 8-byte wire word {4 bytes of payload, epoch}: word w of a slot sits at byte 8 * w (two of them make the
// 16-byte line the standalone kernel writes at once).  An 8-byte word arrives whole.
__device__ __forceinline__ void st_wire_8(void* p, uint32_t payload, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_wire_8(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

}  // namespace awq
