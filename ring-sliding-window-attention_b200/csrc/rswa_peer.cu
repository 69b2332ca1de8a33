// Peer-store halo exchange: the three small device-side pieces of a put / flag protocol between GPUs
// of one node, for halo K/V tiles going forward and their gradients coming back.
//
// The buffers are receiver-owned and mapped into the sender's address space by the caller (symmetric
// memory).  A put is a copy-engine transfer (no SM is taken from the attention kernels) followed by a
// one-thread kernel that releases a sequence number into a flag word next to the buffer; the receiver
// waits for that number with a one-thread kernel on its own compute stream, so that everything launched
// behind it -- kernels that read the landed data from LOCAL memory with ordinary TMA loads -- starts
// after the data is there.  Nothing here loads from a peer, and nothing uses multicast.
//
// The wait is bounded: when the number does not arrive within the given time the kernel raises the
// caller's status word and returns, like every other device-side wait of this library.
//
// Replaces ring_attn_p2p_communicate (ring_swa/ops/comm.py:8-40 of the reference: one NCCL isend and
// irecv per hop, whose kernels run on SMs next to the attention kernels).
#include "rswa_common.cuh"

namespace rswa {
namespace {

constexpr int kErrWaitFlag = 105;

// Sequence numbers only grow; "reached" is wrap-safe.
__device__ __forceinline__ bool reached(int have, int want) { return have - want >= 0; }

__global__ void flag_set_kernel(int* flag, int value) {
  // the copies enqueued ahead of this kernel on the stream have completed; make the order visible
  // system-wide before the number is
  __threadfence_system();
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__global__ void flag_wait_kernel(const int* flag, int value, int* status, unsigned long long timeout_ns) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;  // an error was already reported on this stream
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (reached(v, value)) return;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > timeout_ns) break;
    __nanosleep(200);
  }
  atomicCAS(status, 0, kErrWaitFlag);
}

int check_launch_peer(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace
}  // namespace rswa

using namespace rswa;

extern "C" int rswa_peer_put(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t row_bytes,
                             int64_t rows, int32_t* flag, int32_t value, void* stream_) {
  if (!dst || !src || row_bytes <= 0 || rows <= 0 || dst_pitch < row_bytes || src_pitch < row_bytes) {
    set_error("rswa_peer_put: bad argument");
    return RSWA_E_ARG;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                                    static_cast<size_t>(row_bytes), static_cast<size_t>(rows), cudaMemcpyDeviceToDevice,
                                    stream);
  if (e != cudaSuccess) {
    set_error("rswa_peer_put: cudaMemcpy2DAsync: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  if (flag) {
    flag_set_kernel<<<1, 1, 0, stream>>>(flag, value);
    return check_launch_peer("rswa_peer_put(flag)");
  }
  return RSWA_OK;
}

extern "C" int rswa_flag_set(int32_t* flag, int32_t value, void* stream) {
  if (!flag) {
    set_error("rswa_flag_set: null flag");
    return RSWA_E_ARG;
  }
  flag_set_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, value);
  return check_launch_peer("rswa_flag_set");
}

extern "C" int rswa_flag_wait(const int32_t* flag, int32_t value, int32_t* status, int64_t timeout_ns, void* stream) {
  if (!flag || !status || timeout_ns <= 0) {
    set_error("rswa_flag_wait: flag, status and a positive time limit are required");
    return RSWA_E_ARG;
  }
  flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, value, status,
                                                                  static_cast<unsigned long long>(timeout_ns));
  return check_launch_peer("rswa_flag_wait");
}
