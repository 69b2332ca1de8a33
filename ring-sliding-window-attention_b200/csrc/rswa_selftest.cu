// One 128x128x128 product through each operand path the attention kernels rely on, so that the
// descriptor encodings can be unit-tested in isolation.  See rswa_selftest_mma in include/rswa.h.
#include <cstring>

#include "rswa_common.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;
namespace {

struct SelfCtl {
  uint64_t full, done;
  uint32_t tmem_base;
  int err;
};

__global__ void __launch_bounds__(128, 1)
selftest_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                const uint16_t* __restrict__ a_gmem, float* __restrict__ d, int mode, int swap_lbo_sbo,
                int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kTileBytes;
  SelfCtl* ctl = reinterpret_cast<SelfCtl*>(smem + 2 * kTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&ctl->full, 1);
    mbar_init(&ctl->done, 1);
    ctl->err = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tD = tmem, tA = tmem + 128;
  volatile int* err = &ctl->err;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

  if (mode == 2) {
    // every thread writes its row of A into tensor memory as packed 16-bit pairs
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(a_gmem + (warp * 32 + lane) * 128);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = arow[c * 16 + i];
      tmem_st16(tA + lane_off + c * 16, r);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();

  if (threadIdx.x == 0) {
    mbar_expect_tx(&ctl->full, 2 * kTileBytes);
    tma_load_4d(sA, &a_map, &ctl->full, 0, 0, 0, 0);
    tma_load_4d(sA + kBoxBytes, &a_map, &ctl->full, 64, 0, 0, 0);
    tma_load_4d(sB, &b_map, &ctl->full, 0, 0, 0, 0);
    tma_load_4d(sB + kBoxBytes, &b_map, &ctl->full, 64, 0, 0, 0);
    if (mbar_wait(&ctl->full, 0, err, 1)) {
      tc_fence_after();
      const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
      const uint32_t mn_lbo = swap_lbo_sbo ? 1024 : kBoxBytes;
      const uint32_t mn_sbo = swap_lbo_sbo ? kBoxBytes : 1024;
      for (int k = 0; k < 8; ++k) {
        const uint32_t koff = (k >> 2) * kBoxBytes + (k & 3) * 32;  // K-major: 16 elements along the row
        const uint32_t moff = k * 2048;                             // MN-major: 16 rows down
        const uint32_t acc = k > 0 ? 1u : 0u;
        if (mode == 0) {
          mma_ss(tD, smem_desc_sw128(aA + koff, 16, 1024), smem_desc_sw128(aB + koff, 16, 1024),
                 idesc_f16(128, 128, 1, 0, 0), acc);
        } else if (mode == 1) {
          mma_ss(tD, smem_desc_sw128(aA + koff, 16, 1024), smem_desc_sw128(aB + moff, mn_lbo, mn_sbo),
                 idesc_f16(128, 128, 1, 0, 1), acc);
        } else if (mode == 2) {
          mma_ts(tD, tA + k * 8, smem_desc_sw128(aB + moff, mn_lbo, mn_sbo), idesc_f16(128, 128, 1, 0, 1), acc);
        } else {
          mma_ss(tD, smem_desc_sw128(aA + moff, mn_lbo, mn_sbo), smem_desc_sw128(aB + moff, mn_lbo, mn_sbo),
                 idesc_f16(128, 128, 1, 1, 1), acc);
        }
      }
      mma_commit(&ctl->done);
    }
  }
  bool ok = mbar_wait(&ctl->done, 0, err, 2);
  ok = __all_sync(0xffffffffu, ok);
  tc_fence_after();
  if (ok) {
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tD + lane_off + c * 32, r);
      tmem_ld_wait();
      float* drow = d + (warp * 32 + lane) * 128 + c * 32;
#pragma unroll
      for (int i = 0; i < 32; ++i) drow[i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (threadIdx.x == 0 && ctl->err != 0) atomicCAS(status, 0, ctl->err);
}

}  // namespace
}  // namespace rswa

using namespace rswa;

extern "C" int rswa_selftest_mma(int32_t mode, const void* a, const void* b, float* d, int32_t* status,
                                 void* stream) {
  if (!a || !b || !d || !status) {
    set_error("rswa_selftest_mma: null argument");
    return RSWA_E_ARG;
  }
  const int swap = (mode >> 4) & 1;
  mode &= 15;
  if (mode < 0 || mode > 3) {
    set_error("rswa_selftest_mma: mode must be 0..3");
    return RSWA_E_ARG;
  }
  CUtensorMap am, bm;
  int rc = make_tile_map(&am, a, RSWA_DTYPE_BF16, 1, 128, 1, 128 * 128, 128, 128);
  if (rc) return rc;
  rc = make_tile_map(&bm, b, RSWA_DTYPE_BF16, 1, 128, 1, 128 * 128, 128, 128);
  if (rc) return rc;
  const int smem = 2 * kTileBytes + 1024 + 256;
  cudaError_t e = cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) {
    set_error("rswa_selftest_mma: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(am, bm, static_cast<const uint16_t*>(a), d,
                                                                      mode, swap, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_selftest_mma: launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}
