// A16MatMul, 4-bit weights, decode shapes (M <= 8): y[M,N] = bf16( x[M,K] * dequant(W)[N,K]^T (+ bias) ).
//
// Semantics follow tpu::A16MatMulOp::inference, static w4 path with w_transpose
// (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246): weight bytes [N, K/2] with the even k in
// the low nibble, W[n,k] = (q - zp[n, k/g]) * scale[n, k/g], fp32 accumulation, bf16 output.
//
// The kernel is bound by reading the packed weights once from HBM.  A block of 4 warps owns 16 output rows;
// each warp takes a quarter of K and issues all of its 8-byte weight loads up front.  Nibbles become exact
// bf16 integers with one logic op each ((w >> 4j) & 0x000F000F | 0x43004300 = 128 + q), the zero point is
// removed with one bf16x2 subtract, and the products run on the tensor cores as mma.m16n8k16 (bf16 x bf16,
// fp32 accumulate) with the M tokens in the 8 columns.  Because a dot product does not care about the order
// of k, the activations are staged in shared memory pre-permuted to the nibble order the extraction yields.
// The group scale multiplies the fp32 partial sum of each group, so the only rounding is fp32 accumulation.
#include <cuda_bf16.h>

#include "a16.h"
#include "internal.h"

namespace b200q {
namespace {

constexpr int ROWS_PER_BLOCK = 16;
constexpr int WARPS = 4;
constexpr int CHUNK_K = 64;   // k covered by one 8-byte load per (thread, row): the quad of a row covers 64 k
constexpr int MAX_M = 8;

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// x_perm layout (bf16): row m at m * row_bytes; inside a row, 64-k chunk j at j*128 bytes; inside a chunk,
// quad lane c (k offset c*16) at c*32 bytes, word w (k offset w*8) at w*16 bytes, then the 8 values in nibble
// order (0,4,1,5,2,6,3,7).  row_bytes = 2K + 16 keeps two rows a bank group apart.
__device__ __forceinline__ int xperm_offset_bytes(int k) {
  const int chunk = k >> 6, c = (k >> 4) & 3, w = (k >> 3) & 1, nib = k & 7;
  const int pos = ((nib & 3) << 1) | (nib >> 2);  // 0,4,1,5,2,6,3,7 -> 0..7
  return chunk * 128 + c * 32 + w * 16 + pos * 2;
}

template <int CHUNKS_PER_WARP_BATCH>
__global__ void __launch_bounds__(WARPS * 32)
a16_w4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ wq,
                   const __nv_bfloat16* __restrict__ scale, const uint8_t* __restrict__ zp,
                   const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N, int K, int group) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int row_bytes = 2 * K + 16;
  uint8_t* xs = smem;                                                   // M rows of permuted activations
  float* red = reinterpret_cast<float*>(smem + (size_t)M * row_bytes);  // [WARPS][16 rows][8 cols]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  // ---- stage the activations (bf16, permuted)
  for (int i = tid; i < M * K; i += WARPS * 32) {
    const int m = i / K, k = i - m * K;
    *reinterpret_cast<__nv_bfloat16*>(xs + (size_t)m * row_bytes + xperm_offset_bytes(k)) = x[i];
  }
  __syncthreads();

  const int n0 = blockIdx.x * ROWS_PER_BLOCK;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);  // clamped: rows past N are computed, not stored
  const int chunks = K / CHUNK_K;
  const int chunks_per_warp = (chunks + WARPS - 1) / WARPS;
  const int ch_begin = warp * chunks_per_warp, ch_end = min(chunks, ch_begin + chunks_per_warp);
  const int groups_per_row = K / group;
  const int chunks_per_group = group / CHUNK_K;
  const uint8_t* w0p = wq + (size_t)r0 * (K / 2) + c * 8;
  const uint8_t* w1p = wq + (size_t)r1 * (K / 2) + c * 8;
  const uint8_t* xrow = xs + (size_t)g * row_bytes + c * 32;  // this lane's token (column g of the MMA)
  const bool has_x = g < M;

  float tot[4] = {0.f, 0.f, 0.f, 0.f};
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int cb = ch_begin; cb < ch_end; cb += CHUNKS_PER_WARP_BATCH) {
    uint2 wa[CHUNKS_PER_WARP_BATCH], wb[CHUNKS_PER_WARP_BATCH];
#pragma unroll
    for (int i = 0; i < CHUNKS_PER_WARP_BATCH; ++i) {
      const int ch = min(cb + i, ch_end - 1);
      wa[i] = __ldg(reinterpret_cast<const uint2*>(w0p + (size_t)ch * 32));
      wb[i] = __ldg(reinterpret_cast<const uint2*>(w1p + (size_t)ch * 32));
    }
#pragma unroll
    for (int i = 0; i < CHUNKS_PER_WARP_BATCH; ++i) {
      const int ch = cb + i;
      if (ch >= ch_end) break;
      const int grp = ch / chunks_per_group;
      const uint32_t z0 = zp[(size_t)r0 * groups_per_row + grp], z1 = zp[(size_t)r1 * groups_per_row + grp];
      const uint32_t zc0 = 0x43004300u | z0 | (z0 << 16), zc1 = 0x43004300u | z1 | (z1 << 16);
      uint4 xb0 = make_uint4(0, 0, 0, 0), xb1 = make_uint4(0, 0, 0, 0);
      if (has_x) {
        xb0 = lds128(xrow + ch * 128);
        xb1 = lds128(xrow + ch * 128 + 16);
      }
      const uint32_t wwa[2] = {wa[i].x, wa[i].y}, wwb[2] = {wb[i].x, wb[i].y};
      const uint4 xbs[2] = {xb0, xb1};
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const uint32_t a = wwa[w], b = wwb[w];
        // k-step 0 of this word: nibbles (0,4) -> slots (2c, 2c+1), nibbles (1,5) -> slots (2c+8, 2c+9)
        uint32_t a0 = sub_bf16x2((a & 0x000F000Fu) | 0x43004300u, zc0);
        uint32_t a2 = sub_bf16x2(((a >> 4) & 0x000F000Fu) | 0x43004300u, zc0);
        uint32_t a1 = sub_bf16x2((b & 0x000F000Fu) | 0x43004300u, zc1);
        uint32_t a3 = sub_bf16x2(((b >> 4) & 0x000F000Fu) | 0x43004300u, zc1);
        mma_bf16_16816(acc, a0, a1, a2, a3, xbs[w].x, xbs[w].y);
        // k-step 1: nibbles (2,6) and (3,7)
        a0 = sub_bf16x2(((a >> 8) & 0x000F000Fu) | 0x43004300u, zc0);
        a2 = sub_bf16x2(((a >> 12) & 0x000F000Fu) | 0x43004300u, zc0);
        a1 = sub_bf16x2(((b >> 8) & 0x000F000Fu) | 0x43004300u, zc1);
        a3 = sub_bf16x2(((b >> 12) & 0x000F000Fu) | 0x43004300u, zc1);
        mma_bf16_16816(acc, a0, a1, a2, a3, xbs[w].z, xbs[w].w);
      }
      if ((ch + 1) % chunks_per_group == 0 || ch + 1 == ch_end) {
        // the group (or this warp's part of it) is complete: apply its scale to the fp32 partial sum
        const float s0 = __bfloat162float(scale[(size_t)r0 * groups_per_row + grp]);
        const float s1 = __bfloat162float(scale[(size_t)r1 * groups_per_row + grp]);
        tot[0] = fmaf(acc[0], s0, tot[0]);
        tot[1] = fmaf(acc[1], s0, tot[1]);
        tot[2] = fmaf(acc[2], s1, tot[2]);
        tot[3] = fmaf(acc[3], s1, tot[3]);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      }
    }
  }
  // ---- combine the K quarters of the 4 warps: tot[0..1] = (row g, tokens 2c, 2c+1), tot[2..3] = (row g+8, ..)
  float* mine = red + warp * (16 * 8);
  mine[g * 8 + 2 * c] = tot[0];
  mine[g * 8 + 2 * c + 1] = tot[1];
  mine[(g + 8) * 8 + 2 * c] = tot[2];
  mine[(g + 8) * 8 + 2 * c + 1] = tot[3];
  __syncthreads();
  for (int i = tid; i < 16 * 8; i += WARPS * 32) {
    const int row = i >> 3, m = i & 7;
    const int n = n0 + row;
    if (n < N && m < M) {
      float v = red[i] + red[128 + i] + red[256 + i] + red[384 + i];
      if (bias) v += bias[n];
      y[(size_t)m * N + n] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace

int a16_w4_gemv_supported(int M, int N, int K, int group, const char** why) {
  const char* w = nullptr;
  if (M < 1 || M > MAX_M) w = "M must be in [1, 8]";
  else if (K % CHUNK_K != 0) w = "K must be a multiple of 64";
  else if (group < CHUNK_K || group % CHUNK_K != 0 || K % group != 0) w = "group size must be a multiple of 64 dividing K";
  else if ((size_t)M * (2 * K + 16) + WARPS * 16 * 8 * 4 > 200 * 1024) w = "activations do not fit in shared memory";
  else if (N < 1) w = "empty N";
  if (why) *why = w;
  return w == nullptr;
}

int a16_w4_gemv_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       int M, int N, int K, int group, cudaStream_t stream) {
  const char* why = nullptr;
  if (!a16_w4_gemv_supported(M, N, K, group, &why)) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 gemv: %s", why);
  if ((reinterpret_cast<uintptr_t>(wq) & 7) != 0) return set_error(B200Q_ERR_INVALID, "a16 w4 gemv: weight pointer must be 8-byte aligned");
  const size_t smem = (size_t)M * (2 * K + 16) + WARPS * 16 * 8 * 4;
  auto kfn = a16_w4_gemv_kernel<8>;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int blocks = (N + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  kfn<<<blocks, WARPS * 32, smem, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(wq),
                                            static_cast<const __nv_bfloat16*>(scale), static_cast<const uint8_t*>(zp),
                                            bias, static_cast<__nv_bfloat16*>(y), M, N, K, group);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
