// Tensor-pipe peak probe: every SM issues tcgen05.mma on operand tiles that stay in its shared memory, nothing else.
// The figure it yields is the denominator for the tensor-bound kernels of this library (kind::i8 has no library
// GEMM to measure a peak with); it is a measuring aid with no counterpart in the reference.
//
// One CTA per SM (or one CTA pair per two SMs with cta_group::2).  A: 128 rows x 128 bytes of K, B: 256 rows x 128
// bytes (pair: 128 rows in each CTA), both K-major with the 128-byte swizzle; the content is pseudo-random bytes
// (bf16: finite values near 1) so that the data path toggles as it does in real work.  One thread issues k-blocks of
// four MMAs (128 x 256 x 32 bytes of K each) into two 256-column accumulators alternately, commits every BATCH k-blocks
// and keeps two batches in flight; each wait is bounded.
#include <cstdint>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int PEAK_THREADS = 128;
constexpr int PEAK_BATCH = 8;                 // k-blocks per commit
constexpr uint64_t PEAK_WAIT_NS = 200000000;  // one batch takes microseconds
constexpr uint32_t PEAK_A_BYTES = 128 * 128;
constexpr uint32_t PEAK_B_BYTES = 256 * 128;
constexpr uint32_t PEAK_SMEM = 1024 + PEAK_A_BYTES + PEAK_B_BYTES + 64;

template <bool PAIR, bool BF16>
__global__ void __launch_bounds__(PEAK_THREADS) tc_peak_kernel(int batches, uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* tiles = smem_raw + (base - ptx::smem_u32(smem_raw));
  constexpr uint32_t B_BYTES = PAIR ? PEAK_B_BYTES / 2 : PEAK_B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + PEAK_A_BYTES + PEAK_B_BYTES);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  const int warp = threadIdx.x >> 5;
  const bool leader = !PAIR || ptx::cluster_ctarank() == 0;

  // operand content
  uint32_t* w32 = reinterpret_cast<uint32_t*>(tiles);
  for (uint32_t i = threadIdx.x; i < (PEAK_A_BYTES + B_BYTES) / 4; i += PEAK_THREADS) {
    uint32_t h = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    w32[i] = BF16 ? ((h & 0x807F807Fu) | 0x3F003F00u) : h;
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bars[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&bars[1]), 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::fence_proxy_async_smem();  // the tiles were written through the generic proxy, the MMAs read them through the async one
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(tmem_ptr_smem), 512);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), 512);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (threadIdx.x == 0 && leader) {
    const uint64_t desc0 = ptx::make_smem_desc_kmajor(base, 1024, 2);
    const uint32_t hi = (uint32_t)(desc0 >> 32);
    const uint32_t a_lo = (uint32_t)desc0;
    const uint32_t b_lo = (uint32_t)ptx::make_smem_desc_kmajor(base + PEAK_A_BYTES, 1024, 2);
    uint32_t phase[2] = {0u, 0u};
    int in_flight = 0, slot = 0;
    bool ok = true;
    for (int b = 0; b < batches && ok; ++b) {
      if (in_flight == 2) {
        ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bars[slot]), phase[slot], abort_flag, 1, PEAK_WAIT_NS);
        phase[slot] ^= 1u;
        --in_flight;
        if (!ok) break;
      }
      const uint32_t d = tmem_base + (uint32_t)(b & 1) * 256u;
#pragma unroll
      for (int j = 0; j < PEAK_BATCH; ++j) {
        const uint32_t acc = j != 0 ? 1u : 0u;
        if (PAIR) {
          if (BF16) ptx::umma_kblock_f16_pair(d, a_lo, b_lo, hi, hi, idesc, acc);
          else ptx::umma_kblock_i8_pair(d, a_lo, b_lo, hi, hi, idesc, acc);
        } else {
          if (BF16) ptx::umma_kblock_f16(d, a_lo, b_lo, hi, hi, idesc, acc);
          else ptx::umma_kblock_i8(d, a_lo, b_lo, hi, hi, idesc, acc);
        }
      }
      if (PAIR) ptx::umma_commit_pair(ptx::smem_u32(&bars[slot]), 1);  // signals the leader's barrier only
      else ptx::umma_commit(ptx::smem_u32(&bars[slot]));
      slot ^= 1;
      ++in_flight;
    }
    // drain in issue order; after a timeout the remaining waits are still bounded
    while (in_flight > 0) {
      const int s = in_flight == 2 ? slot : (slot ^ 1);
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars[s]), phase[s], abort_flag, 2, PEAK_WAIT_NS)) break;
      phase[s] ^= 1u;
      --in_flight;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, 512);
    else ptx::tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicCAS(status, 0, *abort_flag);
}

template <bool PAIR, bool BF16>
int launch_peak(int grid, int batches, int launches, int* status, cudaStream_t s) {
  auto kern = tc_peak_kernel<PAIR, BF16>;
  CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PEAK_SMEM));
  const uint32_t idesc = BF16 ? ptx::make_idesc(1u, 1u, 1u, PAIR ? 256u : 128u, 256u)
                              : ptx::make_idesc(2u, 1u, 1u, PAIR ? 256u : 128u, 256u);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(PEAK_THREADS);
  cfg.dynamicSmemBytes = PEAK_SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  for (int i = 0; i < launches; ++i) CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, batches, idesc, status));
  return B200Q_OK;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" int b200q_probe_tensor_peak(int32_t kind, int32_t pair, int32_t kblocks, int32_t launches, double* ms,
                                        double* ops, void* stream) {
  if ((kind != 0 && kind != 1) || kblocks < PEAK_BATCH || kblocks > (1 << 24) || launches < 1 || launches > 100000 || !ms || !ops)
    return set_error(B200Q_ERR_INVALID, "probe_tensor_peak: bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = pair ? (sms / 2) * 2 : sms;
  const int batches = kblocks / PEAK_BATCH;
  int* status = nullptr;
  CUDA_TRY(cudaMalloc(&status, sizeof(int)));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int rc = B200Q_OK;
  int h_status = 0;
  float elapsed = 0.f;
  auto body = [&]() -> int {
    CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));
    CUDA_TRY(cudaEventCreate(&e0));
    CUDA_TRY(cudaEventCreate(&e1));
    auto run = [&](int n) {
      return pair ? (kind ? launch_peak<true, true>(grid, batches, n, status, s) : launch_peak<true, false>(grid, batches, n, status, s))
                  : (kind ? launch_peak<false, true>(grid, batches, n, status, s) : launch_peak<false, false>(grid, batches, n, status, s));
    };
    B200Q_TRY(run(1));  // warm-up launch (module load, clocks)
    CUDA_TRY(cudaEventRecord(e0, s));
    B200Q_TRY(run(launches));
    CUDA_TRY(cudaEventRecord(e1, s));
    CUDA_TRY(cudaEventSynchronize(e1));
    CUDA_TRY(cudaEventElapsedTime(&elapsed, e0, e1));
    CUDA_TRY(cudaMemcpy(&h_status, status, sizeof(int), cudaMemcpyDeviceToHost));
    return B200Q_OK;
  };
  rc = body();
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(status);
  if (rc != B200Q_OK) return rc;
  if (h_status != 0) return set_error(B200Q_ERR_TIMEOUT, "probe_tensor_peak: a bounded wait ran out (site %d)", h_status);
  *ms = (double)elapsed;
  // one k-block = four MMAs of (pair ? 256 : 128) x 256 x (32 bytes of K: 32 int8 or 16 bf16 elements)
  const double k_per_mma = kind ? 16.0 : 32.0;
  const double ctas = pair ? grid / 2 : grid;
  *ops = 2.0 * (pair ? 256.0 : 128.0) * 256.0 * k_per_mma * 4.0 * (double)batches * PEAK_BATCH * ctas * (double)launches;
  return B200Q_OK;
}
