// One-shot sum of the row-parallel partial outputs over peer memory (NVLink / NVSwitch).
//
// A row-sharded linear (down / o projections split along K) leaves one [M, N] fp16 partial per GPU;
// the result is their sum.  At decode sizes (16 KB for one row of N = 8192) a ring or tree collective
// is pure latency: the library all-reduce costs ~65 us on 8 GPUs.  Here every rank reads all peers'
// partials directly with plain peer loads and adds them itself:
//
//   1. ready:  rank r stores the call's epoch into slot [r] of every peer's flag array (system scope,
//              release) - "my partial for this call is written" (the kernel that wrote it precedes
//              this one on the stream);
//   2. wait:   every block polls its OWN flag array until all slots show the epoch (acquire);
//   3. sum:    16-byte peer loads that bypass L1, fp32 adds in rank order (every rank gets identical
//              bits), one fp16 rounding, store to the local output;
//   4. done:   the last block to finish stores the epoch into the peers' done slots and waits for
//              theirs, so that no rank overwrites its partial (next call) while a peer still reads it.
//
// Buffers and flag arrays live in symmetric memory that the caller allocated and exchanged (one
// pointer per rank, as a device array).  The epoch is kept in device memory and advanced by the kernel,
// so the call can be captured in a CUDA graph and replayed.  No multicast / multimem loads are used.
// Every wait is bounded (~2 s); on expiry the kernel sets a status word and returns, and the output of
// that call is invalid.  The ranks must make matching calls: after an expired wait (or any other mismatch
// in the number of calls) the ranks' call counters disagree and every later call expires too, until the flag
// arrays and receive areas have been zeroed again on every rank with no call in flight (a collective reset;
// the wait-limit word may be kept).
#include "awq_peer.cuh"

namespace awq {

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Peer partials are read with L1 bypassed (the same addresses carry new data every call) but as ordinary
// coalescable loads: a warp's 32 x 16 bytes travel as four 128-byte requests.  Volatile loads are issued
// one 16-byte request per thread, and thousands of those per call over NVLink cost hundreds of
// microseconds on 8 GPUs.
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Waits until flags[off + r] == epoch for every r < world.  Returns false on expiry.
__device__ __forceinline__ bool wait_all(const unsigned* flags, int off, int world, unsigned epoch,
                                         unsigned long long limit) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const unsigned long long t0 = clock64();
    while (ld_acquire_sys(flags + off + threadIdx.x) != epoch) {
      if (clock64() - t0 > limit) { s_ok = 0; break; }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

constexpr int kArThreads = 256;

__global__ void __launch_bounds__(kArThreads)
peer_allreduce_kernel(const uint16_t* const* bufs, unsigned* const* flags, uint16_t* out, const uint16_t* bias,
                      size_t count, int ncols, int rank, int world) {
  // Launched with programmatic stream serialization: this grid may start while the kernel that writes the
  // partial is still finishing, and the next kernel of the stream may start (and prefetch its weights) while
  // this one waits for the peers.  Nothing below touches memory before the previous kernel has completed.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  unsigned* my_flags = flags[rank];
  const unsigned epoch = my_flags[kArEpochOff] + 1u;   // written only by this kernel's last block, a launch ago
  const unsigned long long limit = wait_limit_cycles(my_flags);
  if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(flags[threadIdx.x] + kArReadyOff + rank, epoch);
  const bool ready = wait_all(my_flags, kArReadyOff, world, epoch, limit);
  if (!ready && threadIdx.x == 0) atomicCAS(my_flags + kArStatusOff, 0u, 1u);

  if (ready) {
    const size_t vecs = count / 8;                       // 8 halves per 16-byte load
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      uint4 v[kArMaxWorld];
#pragma unroll
      for (int r = 0; r < kArMaxWorld; ++r)
        if (r < world) v[r] = ld_peer_16(bufs[r] + i * 8);
#pragma unroll
      for (int r = 0; r < kArMaxWorld; ++r) {
        if (r < world) {
          const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            acc[2 * e] += f.x;
            acc[2 * e + 1] += f.y;
          }
        }
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
      if (bias != nullptr) {
        const size_t col = (i * 8) % static_cast<size_t>(ncols);
        const uint4 b = *reinterpret_cast<const uint4*>(bias + col);
        const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __hadd2(oh[e], bh[e]);
      }
      *reinterpret_cast<uint4*>(out + i * 8) = o;
    }
  }

  // The last block to get here tells the peers that this rank has read their partials, waits for the
  // same from them, and closes the call.
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(my_flags + kArBlocksOff, 1u);
    s_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < world) st_release_sys(flags[threadIdx.x] + kArDoneOff + rank, epoch);
  const bool done = wait_all(my_flags, kArDoneOff, world, epoch, limit);
  if (threadIdx.x == 0) {
    if (!done) atomicCAS(my_flags + kArStatusOff, 0u, 2u);
    my_flags[kArBlocksOff] = 0u;
    my_flags[kArEpochOff] = epoch;
  }
}

// ---------------------------------------------------------------------------------------------------
// Push variant.  Instead of publishing a flag and letting the peers pull the partial (a flag's one-way trip
// followed by a load's round trip over NVLink), every rank stores its partial into a receive slot on each
// peer, and the data carries its own flag: each 8-byte word on the wire is {4 bytes of payload, the call's
// epoch}, written with 16-byte stores of two such words.  An 8-byte word arrives whole, so a receiver polls
// its own memory until both words of a 16-byte line show the current epoch and then owns the payload: no
// fence, no separate flag, one one-way trip.  The wire format doubles the bytes, which at these sizes
// (16 KB ... 1 MB per rank) costs less than a second trip.
//
// There is no "done" phase.  The receive slots are double-buffered on the parity of the call's epoch (kept
// in device memory, so captured graphs replay correctly): a rank overwrites slot [e & 1] in call e + 2, which
// it can reach only after finishing call e + 1, which it finished only after receiving every peer's words of
// call e + 1, which a peer sends only after its own call e has completed (calls on a stream do not overlap:
// each kernel of the chain waits for its predecessor before touching anything).
// ---------------------------------------------------------------------------------------------------
// recv[r]: rank r's receive area, 2 parities x world slots x (4 * slot_elems) bytes (wire format).
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_push_kernel(const uint16_t* partial, unsigned char* const* recv, unsigned* const* flags, uint16_t* out,
                           const uint16_t* bias, size_t count, int ncols, size_t slot_elems, int rank, int world) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ int s_ok;
  unsigned* my_flags = flags[rank];
  const unsigned epoch = my_flags[kArPushEpochOff] + 1u;   // written only by this kernel's last block, a launch ago
  const unsigned long long limit = wait_limit_cycles(my_flags);
  const size_t slot_bytes = slot_elems * 4;
  const size_t par_off = static_cast<size_t>(epoch & 1u) * world;
  const size_t vecs = count / 8;
  const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();

  // 1. this thread's vectors of the partial go to every peer's slot [parity][rank], two wire lines each
  for (size_t i = first; i < vecs; i += stride) {
    const uint4 v = *reinterpret_cast<const uint4*>(partial + i * 8);
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r) {
      if (r < world && r != rank) {
        unsigned char* dst = recv[r] + (par_off + rank) * slot_bytes + i * 32;
        st_wire_16(dst, v.x, v.y, epoch);
        st_wire_16(dst + 16, v.z, v.w, epoch);
      }
    }
  }

  // 2. the same vectors of every peer, polled out of this rank's own memory, summed in rank order
  // One limit for the whole call: once a wait has run out (in this thread or, seen through s_ok, in another
  // thread of the block) no further word is polled, so a call returns about one limit after it started.
  const unsigned char* slots = recv[rank] + par_off * slot_bytes;
  volatile int* block_ok = &s_ok;
  const unsigned long long t_call = clock64();
  for (size_t i = first; i < vecs; i += stride) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    bool ok = true;
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r) {
      if (r < world && ok) {
        uint4 v;
        if (r == rank) {
          v = *reinterpret_cast<const uint4*>(partial + i * 8);
        } else {
          const unsigned char* src = slots + static_cast<size_t>(r) * slot_bytes + i * 32;
          uint4 a = ld_wire_16(src), b = ld_wire_16(src + 16);
          unsigned spins = 0;
          while (a.y != epoch || a.w != epoch || b.y != epoch || b.w != epoch) {
            if ((++spins & 15u) == 0u && (*block_ok == 0 || clock64() - t_call > limit)) { ok = false; break; }
            a = ld_wire_16(src);
            b = ld_wire_16(src + 16);
          }
          v = make_uint4(a.x, a.z, b.x, b.z);
        }
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
    if (!ok) { s_ok = 0; break; }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
    if (bias != nullptr) {
      const size_t col = (i * 8) % static_cast<size_t>(ncols);
      const uint4 bv = *reinterpret_cast<const uint4*>(bias + col);
      const __half2* bh = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __hadd2(oh[e], bh[e]);
    }
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }

  // 3. the last block closes the call
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_ok == 0) atomicCAS(my_flags + kArStatusOff, 0u, 3u);
    const unsigned prev = atomicAdd(my_flags + kArPushBlocksOff, 1u);
    if (prev == gridDim.x - 1) {
      my_flags[kArPushBlocksOff] = 0u;
      my_flags[kArPushEpochOff] = epoch;
    }
  }
}

}  // namespace awq

extern "C" {

size_t awq_b200_peer_allreduce_flag_bytes(void) { return awq::kArFlagWords * sizeof(unsigned); }

// bufs / flags: device arrays of `world` pointers (this rank's own at index `rank`).  `count` fp16 elements,
// a multiple of 8; every buffer 16-byte aligned.  `bias` (optional, [ncols]) is added after the sum.
int awq_b200_peer_allreduce(const void* const* bufs, void* const* flags, void* out, const void* bias, size_t count,
                            int ncols, int rank, int world, awq_b200_stream_t stream) {
  using namespace awq;
  if (!bufs || !flags || !out) return AWQ_B200_ERR_NULL;
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return AWQ_B200_ERR_SHAPE;
  if (count == 0 || (count % 8) != 0 || (bias && (ncols < 8 || (ncols % 8) != 0))) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(out) || (bias && !aligned16(bias))) return AWQ_B200_ERR_ALIGN;
  const size_t vecs = count / 8;
  int blocks = static_cast<int>((vecs + kArThreads - 1) / kArThreads);
  if (blocks > 64) blocks = 64;        // all blocks must be resident together: they wait on one another's peers
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, reinterpret_cast<const uint16_t* const*>(bufs),
                                  reinterpret_cast<unsigned* const*>(flags), static_cast<uint16_t*>(out),
                                  static_cast<const uint16_t*>(bias), count, ncols, rank, world));
  return AWQ_B200_OK;
}

// Push variant: `partial` is this rank's [count] fp16 partial (any device memory of this GPU); `recv` is a device
// array of `world` pointers to the ranks' receive areas of 2 * world * slot_elems * 4 bytes each (peer-mapped
// memory, zero before the first call; slot_elems >= count, a multiple of 8); `flags` as above.
int awq_b200_peer_allreduce_push(const void* partial, void* const* recv, void* const* flags, void* out, const void* bias,
                                 size_t count, int ncols, size_t slot_elems, int rank, int world,
                                 awq_b200_stream_t stream) {
  using namespace awq;
  if (!partial || !recv || !flags || !out) return AWQ_B200_ERR_NULL;
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return AWQ_B200_ERR_SHAPE;
  if (count == 0 || (count % 8) != 0 || slot_elems < count || (slot_elems % 8) != 0 ||
      (bias && (ncols < 8 || (ncols % 8) != 0)))
    return AWQ_B200_ERR_SHAPE;
  if (!aligned16(partial) || !aligned16(out) || (bias && !aligned16(bias))) return AWQ_B200_ERR_ALIGN;
  const size_t vecs = count / 8;
  int blocks = static_cast<int>((vecs + kArThreads - 1) / kArThreads);
  if (blocks > kArMaxBlocks) blocks = kArMaxBlocks;   // one flag per block and peer; all blocks resident together
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AWQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_allreduce_push_kernel, static_cast<const uint16_t*>(partial),
                                  reinterpret_cast<unsigned char* const*>(recv), reinterpret_cast<unsigned* const*>(flags),
                                  static_cast<uint16_t*>(out), static_cast<const uint16_t*>(bias), count, ncols,
                                  slot_elems, rank, world));
  return AWQ_B200_OK;
}

}  // extern "C"
