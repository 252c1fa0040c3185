// A16MatMul, 4-bit weights, decode shapes (M <= 8): y[M,N] = bf16( x[M,K] * dequant(W)[N,K]^T (+ bias) ).
//
// Semantics follow tpu::A16MatMulOp::inference, static w4 path with w_transpose
// (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246): weight bytes [N, K/2] with the even k in
// the low nibble, W[n,k] = (q - zp[n, k/g]) * scale[n, k/g], fp32 accumulation, bf16 output.
//
// The kernel is bound by reading the packed weights once from HBM.  It is persistent: one block per SM walks
// slabs of 16 output rows (a contiguous 16 * K/2 byte piece of the weight matrix).  A producer warp streams
// slabs into a shared-memory ring with bulk copies (cp.async.bulk, one per slab) plus the slab's
// scales and zero points, running ahead of the 16 consumer warps, which split K.  The activations are staged
// in shared memory once per block.  Nibbles become exact bf16 integers with one logic op each
// ((w >> 4j) & 0x000F000F | 0x43004300 = 128 + q), 128 + zero point is removed with one bf16x2 fma, and the
// products run on the tensor cores as mma.m16n8k16 (bf16 x bf16, fp32 accumulate) with the M tokens in the 8
// columns.  Because a dot product does not care about the order of k, the activations are stored pre-permuted
// to the nibble order the extraction yields.  The group scale multiplies the fp32 partial sum of each group,
// so the only rounding is fp32 accumulation.  Every wait is bounded; a wait that runs out sets *status.
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "a16.h"
#include "devbuf.h"
#include "internal.h"
#include "ptx_sm100.cuh"
#include "round16.cuh"

namespace b200q {
namespace {

constexpr int ROWS = 16;           // rows per slab = M of the MMA
constexpr int CWARPS = 16;         // consumer warps (split K)
constexpr int THREADS = (CWARPS + 1) * 32;
constexpr int CHUNK_K = 64;        // k covered by one 8-byte load per (lane, row): the quad of a row covers 64 k
constexpr int MAX_M = 8;
constexpr int MAX_STAGES = 4;
constexpr uint64_t WAIT_NS = 2000000000ull;

// a - b on packed bf16 as one fused multiply-add a * 1.0 + (-b) (exact here: small integers)
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(0x3F803F80u), "r"(b ^ 0x80008000u));
  return d;
}

// acc += a.lo * b.lo + a.hi * b.hi for packed bf16 pairs, fp32 accumulate (mixed-precision FMA: the bf16 halves are
// read in place, products are exact, one rounding per addition)
__device__ __forceinline__ void fma2_f32_bf16(float& acc, uint32_t a, uint32_t b) {
  asm("{\n\t"
      ".reg .b16 al, ah, bl, bh;\n\t"
      "mov.b32 {al, ah}, %1;\n\t"
      "mov.b32 {bl, bh}, %2;\n\t"
      "fma.rn.f32.bf16 %0, al, bl, %0;\n\t"
      "fma.rn.f32.bf16 %0, ah, bh, %0;\n\t"
      "}"
      : "+f"(acc)
      : "r"(a), "r"(b));
}

// the same with IEEE half operands
__device__ __forceinline__ void fma2_f32_f16(float& acc, uint32_t a, uint32_t b) {
  asm("{\n\t"
      ".reg .b16 al, ah, bl, bh;\n\t"
      "mov.b32 {al, ah}, %1;\n\t"
      "mov.b32 {bl, bh}, %2;\n\t"
      "fma.rn.f32.f16 %0, al, bl, %0;\n\t"
      "fma.rn.f32.f16 %0, ah, bh, %0;\n\t"
      "}"
      : "+f"(acc)
      : "r"(a), "r"(b));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x_perm layout (bf16): row m at m * row_bytes; inside a row, the 8 values k0..k0+7 (k0 % 8 == 0) sit at
// (k0 / 64) * 128 + ((k0 / 16) % 4) * 32 + ((k0 / 8) % 2) * 16 bytes in nibble order (0,4,1,5,2,6,3,7): exactly the
// 16 bytes one lane needs for the two MMAs of one packed 32-bit weight word.  row_bytes = 2K + 16 keeps two
// rows a bank group apart.
__device__ __forceinline__ int xperm_offset_bytes8(int k0) {
  return (k0 >> 6) * 128 + ((k0 >> 4) & 3) * 32 + ((k0 >> 3) & 1) * 16;
}

// Shared-memory plan, identical on host and device.
struct GemvPlan {
  int w_pitch;        // weight row pitch in shared memory (dense; the 4-way bank conflict of the 8-byte fragment
                      // loads costs far less than issuing one small bulk copy per row)
  int gpr;            // groups per row
  int scale_off;      // inside a stage: weights | scales (bf16) | zero points
  int zp_off;
  int stage_bytes;
  int x_off, red_off, bar_off, total;
  int stages;
};
// K: the k range a launch covers; KT: the length of the rows it is a part of (the scales and zero points of WHOLE rows are
// staged - a slab's are contiguous in global memory only then - and indexed from the range's first group)
__host__ __device__ inline GemvPlan gemv_plan(int M, int K, int group, bool x_in_smem = true, int KT = 0) {
  GemvPlan p;
  p.w_pitch = K / 2;  // dense: the slab is one contiguous piece of global memory and arrives as ONE bulk copy
  p.gpr = (KT > 0 ? KT : K) / group;
  p.scale_off = ROWS * p.w_pitch;
  p.zp_off = p.scale_off + ((ROWS * p.gpr * 2 + 15) & ~15);
  p.stage_bytes = (p.zp_off + ROWS * p.gpr + 127) & ~127;
  const int x_bytes = x_in_smem ? ((M * (2 * K + 16) + 127) & ~127) : 0;  // the CUDA-core kernel keeps x in registers
  const int red_bytes = 2 * CWARPS * ROWS * 8 * 4;
  const int fixed = x_bytes + red_bytes + 128;
  int st = (220 * 1024 - fixed) / p.stage_bytes;
  p.stages = st > MAX_STAGES ? MAX_STAGES : st;
  p.x_off = p.stages * p.stage_bytes;
  p.red_off = p.x_off + x_bytes;
  p.bar_off = p.red_off + red_bytes;
  p.total = p.bar_off + 128;
  return p;
}

// Producer warp of both decode kernels: streams 16-row weight slabs (one bulk copy each) plus the slab's scales
// and zero points into the shared-memory ring, running ahead of the consumer warps.
// K is the length of the k range this launch covers, starting at k0 of rows that are KT long (K = KT, k0 = 0: the whole
// row; otherwise a slab's rows are 16 separate pieces, one bulk copy each; the scales / zero points of the whole rows are
// staged either way, contiguous in global memory).
__device__ __forceinline__ void gemv_producer(uint8_t* smem, const GemvPlan& P, uint32_t bar_base, volatile int* abort_flag,
                                              const uint8_t* __restrict__ wq, const __nv_bfloat16* __restrict__ scale,
                                              const uint8_t* __restrict__ zp, int N, int K, int num_slabs, int lane,
                                              int KT, int k0, int group) {
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  int stage = 0;
  uint32_t phase = 0;
  for (int slab = blockIdx.x; slab < num_slabs; slab += gridDim.x) {
    bool ok = true;
    if (lane == 0) ok = ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, 1, WAIT_NS);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) break;
    uint8_t* st = smem + (size_t)stage * P.stage_bytes;
    const int n0 = slab * ROWS;
    const int rows = min(ROWS, N - n0);
    __nv_bfloat16* ss = reinterpret_cast<__nv_bfloat16*>(st + P.scale_off);
    uint8_t* sz = st + P.zp_off;
    // scales and zero points of the slab are contiguous in global memory (rows are adjacent)
    const int nmeta = rows * P.gpr;
    const __nv_bfloat16* gs = scale + (size_t)n0 * P.gpr;
    const uint8_t* gz = zp + (size_t)n0 * P.gpr;
    const bool meta_bulk = (nmeta % 16 == 0) && ((reinterpret_cast<uintptr_t>(gs) & 15) == 0) &&
                           ((reinterpret_cast<uintptr_t>(gz) & 15) == 0);
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(full_bar(stage), (uint32_t)rows * (uint32_t)(K / 2) + (meta_bulk ? (uint32_t)nmeta * 3u : 0u));
      if (K == KT) ptx::bulk_load_1d(ptx::smem_u32(st), wq + (size_t)n0 * (K / 2), (uint32_t)rows * (uint32_t)(K / 2), full_bar(stage));
      if (meta_bulk) {
        ptx::bulk_load_1d(ptx::smem_u32(ss), gs, (uint32_t)nmeta * 2u, full_bar(stage));
        ptx::bulk_load_1d(ptx::smem_u32(sz), gz, (uint32_t)nmeta, full_bar(stage));
      }
    }
    if (K != KT) {   // a k range of longer rows: one bulk copy per row piece (the byte count is registered above)
      __syncwarp();
      if (lane < rows)
        ptx::bulk_load_1d(ptx::smem_u32(st + (size_t)lane * (K / 2)), wq + (size_t)(n0 + lane) * (KT / 2) + (k0 >> 1), (uint32_t)(K / 2),
                          full_bar(stage));
    }
    if (!meta_bulk) {  // ragged tail or unaligned metadata: plain loads, all issued before the stores
      for (int i0 = 0; i0 < nmeta; i0 += 32 * 8) {
        __nv_bfloat16 tv[8];
        uint8_t tz[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = i0 + j * 32 + lane;
          if (i < nmeta) {
            tv[j] = gs[i];
            tz[j] = gz[i];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = i0 + j * 32 + lane;
          if (i < nmeta) {
            ss[i] = tv[j];
            sz[i] = tz[j];
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(full_bar(stage));  // second arrival of the phase: metadata is in place
    if (++stage == P.stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
a16_w4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ wq,
                   const __nv_bfloat16* __restrict__ scale, const uint8_t* __restrict__ zp,
                   const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N, int K, int group,
                   int early_weights, int* __restrict__ status, int KT, int k_first, int pass_mode, float* __restrict__ ws) {
  // K: the k range of this launch (k_first .. k_first + K of rows KT long).  pass_mode bit 0: add the partial sums in ws (an earlier
  // range of k) first; bit 1: this is not the last range - leave the fp32 sums in ws instead of rounding them into y.
  extern __shared__ __align__(128) uint8_t smem[];
  const GemvPlan P = gemv_plan(M, K, group, true, KT);
  const int g_first = k_first / group;   // the staged metadata covers whole rows
  // Programmatic dependent launch: the next kernel of the stream may take an SM as soon as this block has left it; when
  // the caller vouches that the weights are constant, the producer requests them before waiting for the predecessor.
  ptx::griddep_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_base = ptx::smem_u32(smem + P.bar_off);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P.bar_off + 16 * MAX_STAGES);
  const int num_slabs = (N + ROWS - 1) / ROWS;
  const int row_bytes = 2 * K + 16;

  if (tid == 0) {
    for (int s = 0; s < P.stages; ++s) {
      ptx::mbar_init(full_bar(s), 2);  // bulk-copy issue (with byte count) + metadata ready
      ptx::mbar_init(empty_bar(s), CWARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();

  if (warp == CWARPS) {
    if (!early_weights) ptx::griddep_wait();
    gemv_producer(smem, P, bar_base, abort_flag, wq, scale, zp, N, K, num_slabs, lane, KT, k_first, group);
  } else {
    // ------------------------------------------------------------ consumer warps
    ptx::griddep_wait();   // activations are read and outputs written only after the predecessor has finished
    uint8_t* xs = smem + P.x_off;
    // stage the activations once per block (bf16, 8 values per 16-byte move, permuted to nibble order)
    const int kv = K / 8;
    for (int i = tid; i < M * kv; i += CWARPS * 32) {
      const int m = i / kv, k0 = (i - m * kv) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * KT + k_first + k0);
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);  // (k0, k4)
      o.y = __byte_perm(v.x, v.z, 0x7632);  // (k1, k5)
      o.z = __byte_perm(v.y, v.w, 0x5410);  // (k2, k6)
      o.w = __byte_perm(v.y, v.w, 0x7632);  // (k3, k7)
      *reinterpret_cast<uint4*>(xs + (size_t)m * row_bytes + xperm_offset_bytes8(k0)) = o;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory");

    const int g = lane >> 2, c = lane & 3;
    const int chunks = K / CHUNK_K;
    const int cpw = (chunks + CWARPS - 1) / CWARPS;
    const int ch_begin = min(warp * cpw, chunks), ch_end = min(chunks, ch_begin + cpw);
    const int cpg = group / CHUNK_K;  // chunks per group
    const uint8_t* xrow = xs + (size_t)g * row_bytes + c * 32;  // this lane's token (column g of the MMA)
    const bool has_x = g < M;
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int slab = blockIdx.x; slab < num_slabs; slab += gridDim.x, ++it) {
      if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, 2, WAIT_NS)) break;
      const uint8_t* st = smem + (size_t)stage * P.stage_bytes;
      const int n0 = slab * ROWS;
      const int rows = min(ROWS, N - n0);
      const int rl0 = min(g, rows - 1), rl1 = min(g + 8, rows - 1);  // rows past N are computed from a valid row, not stored
      const uint8_t* w0p = st + (size_t)rl0 * P.w_pitch + c * 8;
      const uint8_t* w1p = st + (size_t)rl1 * P.w_pitch + c * 8;
      const __nv_bfloat16* sc0 = reinterpret_cast<const __nv_bfloat16*>(st + P.scale_off) + rl0 * P.gpr;
      const __nv_bfloat16* sc1 = reinterpret_cast<const __nv_bfloat16*>(st + P.scale_off) + rl1 * P.gpr;
      const uint8_t* zp0 = st + P.zp_off + rl0 * P.gpr;
      const uint8_t* zp1 = st + P.zp_off + rl1 * P.gpr;
      float tot[4] = {0.f, 0.f, 0.f, 0.f};
      float acc[4][4] = {};  // one accumulator per k-step of a chunk: four independent MMA chains
      int grp = ch_begin / cpg, in_grp = ch_begin - grp * cpg;
      grp += g_first;
      uint32_t z0 = zp0[grp], z1 = zp1[grp];
      uint32_t zc0 = __byte_perm(z0, 0x43u, 0x4040), zc1 = __byte_perm(z1, 0x43u, 0x4040);  // bf16x2 (128 + zp)
#pragma unroll 4
      for (int ch = ch_begin; ch < ch_end; ++ch) {
        const uint2 wa = *reinterpret_cast<const uint2*>(w0p + ch * 32);
        const uint2 wb = *reinterpret_cast<const uint2*>(w1p + ch * 32);
        uint4 xb0 = make_uint4(0, 0, 0, 0), xb1 = make_uint4(0, 0, 0, 0);
        if (has_x) {
          xb0 = *reinterpret_cast<const uint4*>(xrow + ch * 128);
          xb1 = *reinterpret_cast<const uint4*>(xrow + ch * 128 + 16);
        }
        const uint32_t wwa[2] = {wa.x, wa.y}, wwb[2] = {wb.x, wb.y};
        const uint4 xbs[2] = {xb0, xb1};
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const uint32_t a = wwa[w], b = wwb[w];
          const uint32_t a4 = a >> 4, a8 = a >> 8, a12 = a >> 12;
          const uint32_t b4 = b >> 4, b8 = b >> 8, b12 = b >> 12;
          // k-step 0 of this word: nibbles (0,4) -> slots (2c, 2c+1), nibbles (1,5) -> slots (2c+8, 2c+9)
          uint32_t a0 = sub_bf16x2((a & 0x000F000Fu) | 0x43004300u, zc0);
          uint32_t a2 = sub_bf16x2((a4 & 0x000F000Fu) | 0x43004300u, zc0);
          uint32_t a1 = sub_bf16x2((b & 0x000F000Fu) | 0x43004300u, zc1);
          uint32_t a3 = sub_bf16x2((b4 & 0x000F000Fu) | 0x43004300u, zc1);
          mma_bf16_16816(acc[2 * w], a0, a1, a2, a3, xbs[w].x, xbs[w].y);
          // k-step 1: nibbles (2,6) and (3,7)
          a0 = sub_bf16x2((a8 & 0x000F000Fu) | 0x43004300u, zc0);
          a2 = sub_bf16x2((a12 & 0x000F000Fu) | 0x43004300u, zc0);
          a1 = sub_bf16x2((b8 & 0x000F000Fu) | 0x43004300u, zc1);
          a3 = sub_bf16x2((b12 & 0x000F000Fu) | 0x43004300u, zc1);
          mma_bf16_16816(acc[2 * w + 1], a0, a1, a2, a3, xbs[w].z, xbs[w].w);
        }
        if (++in_grp == cpg || ch + 1 == ch_end) {
          // the group (or this warp's part of it) is complete: apply its scale to the fp32 partial sum
          const float s0 = __bfloat162float(sc0[grp]), s1 = __bfloat162float(sc1[grp]);
          float sum4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sum4[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
            acc[0][j] = acc[1][j] = acc[2][j] = acc[3][j] = 0.f;
          }
          tot[0] = fmaf(sum4[0], s0, tot[0]);
          tot[1] = fmaf(sum4[1], s0, tot[1]);
          tot[2] = fmaf(sum4[2], s1, tot[2]);
          tot[3] = fmaf(sum4[3], s1, tot[3]);
          in_grp = 0;
          ++grp;
          if (ch + 1 < ch_end) {
            z0 = zp0[grp];
            z1 = zp1[grp];
            zc0 = __byte_perm(z0, 0x43u, 0x4040);
            zc1 = __byte_perm(z1, 0x43u, 0x4040);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(empty_bar(stage));  // this warp no longer reads the stage
      if (++stage == P.stages) {
        stage = 0;
        phase ^= 1u;
      }
      // ---- combine the K parts of the warps: tot[0..1] = (row g, tokens 2c, 2c+1), tot[2..3] = (row g+8, ..)
      float* mine = red + (size_t)(it & 1) * (CWARPS * ROWS * 8) + warp * (ROWS * 8);
      mine[g * 8 + 2 * c] = tot[0];
      mine[g * 8 + 2 * c + 1] = tot[1];
      mine[(g + 8) * 8 + 2 * c] = tot[2];
      mine[(g + 8) * 8 + 2 * c + 1] = tot[3];
      asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory");
      if (tid < ROWS * 8) {
        const int row = tid >> 3, m = tid & 7;
        const int n = n0 + row;
        if (n < N && m < M) {
          const float* rb = red + (size_t)(it & 1) * (CWARPS * ROWS * 8) + tid;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < CWARPS; ++w) v += rb[w * (ROWS * 8)];
          if (pass_mode & 1) v += ws[(size_t)m * N + n];
          if (pass_mode & 2) {
            ws[(size_t)m * N + n] = v;
          } else {
            if (bias) v += bias[n];
            y[(size_t)m * N + n] = __ushort_as_bfloat16(f32_to_bf16_bits_ref(v));
          }
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && status != nullptr) atomicCAS(status, 0, *abort_flag);
}


// ---------------------------------------------------------------------------------------------------------------
// Resident form of the kernel above for shapes whose whole weight slice fits in shared memory (N = 11008, K = 4096 on
// 148 SMs: five 16-row slabs of 35 KB per block).  The time of a decode call is the latency of its first bytes plus the
// barriers between slabs, not its arithmetic, so here
//   * the producer warp requests EVERY slab of the block at once when the kernel starts (no ring, no empty barriers):
//     the HBM system has the block's whole slice in flight from the first microsecond;
//   * a consumer warp keeps its activations (its 1/16 of K for its token) in registers, read once from global memory, so
//     shared memory holds nothing but weights and the per-slab loop has no shared read of x;
//   * the K parts of the 16 warps are combined once per slab at the END, when every slab's sums sit in registers: the
//     per-slab barrier of the ring form, which serialised 4-chunk work items behind a 512-thread barrier, is gone from
//     the part of the kernel that waits for memory.
constexpr int RES_MAX_SLABS = 6;   // slabs a block may own
constexpr int RES_MAX_CPW = 4;     // 64-k chunks per warp whose activations stay in registers (K <= 4096)

struct ResidentPlan {
  int gpr, scale_off, zp_off, stage_bytes, red_off, bar_off, total;
};
// red_planes: buffers of 16 warps x 128 partial sums for the final combination: one per slab (a single barrier) when
// they fit, else two used in turn (a barrier per slab)
__host__ __device__ inline ResidentPlan resident_plan(int K, int group, int slabs_per_block, int red_planes = 2) {
  ResidentPlan p;
  p.gpr = K / group;
  p.scale_off = ROWS * (K / 2);
  p.zp_off = p.scale_off + ((ROWS * p.gpr * 2 + 15) & ~15);
  p.stage_bytes = (p.zp_off + ROWS * p.gpr + 127) & ~127;
  p.red_off = slabs_per_block * p.stage_bytes;
  p.bar_off = p.red_off + red_planes * CWARPS * ROWS * 8 * 4;
  p.total = p.bar_off + 128;
  return p;
}

__global__ void __launch_bounds__(THREADS, 1)
a16_w4_gemv_resident_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ wq,
                            const __nv_bfloat16* __restrict__ scale, const uint8_t* __restrict__ zp,
                            const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N, int K, int group,
                            int slabs_per_block, int red_planes, int early_weights, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const ResidentPlan P = resident_plan(K, group, slabs_per_block, red_planes);
  // Programmatic dependent launch: the next kernel of the stream may take an SM as soon as this block has left it; when
  // the caller vouches that the weights are constant, this block requests them before it waits for its predecessor.
  ptx::griddep_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_base = ptx::smem_u32(smem + P.bar_off);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P.bar_off + 8 * RES_MAX_SLABS);
  const int num_slabs = (N + ROWS - 1) / ROWS;
  // this block's slabs: blockIdx.x, + gridDim.x, ...
  int nsl = 0;
  for (int sl = blockIdx.x; sl < num_slabs && nsl < slabs_per_block; sl += gridDim.x) ++nsl;

  if (tid == 0) {
    for (int s = 0; s < RES_MAX_SLABS; ++s) ptx::mbar_init(full_bar(s), 2);  // bulk-copy issue (with byte count) + metadata ready
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();

  if (warp == CWARPS) {
    // ---- producer: every slab at once
    if (!early_weights) ptx::griddep_wait();
    for (int s = 0; s < nsl; ++s) {
      const int slab = blockIdx.x + s * gridDim.x;
      uint8_t* st = smem + (size_t)s * P.stage_bytes;
      const int n0 = slab * ROWS;
      const int rows = min(ROWS, N - n0);
      const int nmeta = rows * P.gpr;
      const __nv_bfloat16* gs = scale + (size_t)n0 * P.gpr;
      const uint8_t* gz = zp + (size_t)n0 * P.gpr;
      __nv_bfloat16* ss = reinterpret_cast<__nv_bfloat16*>(st + P.scale_off);
      uint8_t* sz = st + P.zp_off;
      const bool meta_bulk = (nmeta % 16 == 0) && ((reinterpret_cast<uintptr_t>(gs) & 15) == 0) && ((reinterpret_cast<uintptr_t>(gz) & 15) == 0);
      if (lane == 0) {
        ptx::mbar_arrive_expect_tx(full_bar(s), (uint32_t)rows * (uint32_t)(K / 2) + (meta_bulk ? (uint32_t)nmeta * 3u : 0u));
        ptx::bulk_load_1d(ptx::smem_u32(st), wq + (size_t)n0 * (K / 2), (uint32_t)rows * (uint32_t)(K / 2), full_bar(s));
        if (meta_bulk) {
          ptx::bulk_load_1d(ptx::smem_u32(ss), gs, (uint32_t)nmeta * 2u, full_bar(s));
          ptx::bulk_load_1d(ptx::smem_u32(sz), gz, (uint32_t)nmeta, full_bar(s));
        }
      }
      if (!meta_bulk) {  // ragged tail or unaligned metadata: plain loads
        for (int i = lane; i < nmeta; i += 32) {
          ss[i] = gs[i];
          sz[i] = gz[i];
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(full_bar(s));  // second arrival: metadata is in place
    }
  } else {
    // ------------------------------------------------------------ consumer warps
    ptx::griddep_wait();   // activations are read and outputs written only after the predecessor has finished
    const int g = lane >> 2, c = lane & 3;
    const int chunks = K / CHUNK_K;
    const int cpw = (chunks + CWARPS - 1) / CWARPS;   // <= RES_MAX_CPW (host)
    const int ch_begin = min(warp * cpw, chunks), ch_end = min(chunks, ch_begin + cpw);
    const int cpg = group / CHUNK_K;
    // this lane's activations: token g, k in [64 ch + 16 c, + 16) of each of the warp's chunks, in nibble-pair order
    uint4 xr[RES_MAX_CPW][2];
#pragma unroll
    for (int i = 0; i < RES_MAX_CPW; ++i) {
      xr[i][0] = xr[i][1] = make_uint4(0, 0, 0, 0);
      const int ch = ch_begin + i;
      if (g < M && ch < ch_end) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)g * K + (size_t)ch * CHUNK_K + c * 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 v = __ldg(src + h);
          xr[i][h].x = __byte_perm(v.x, v.z, 0x5410);  // (k0, k4)
          xr[i][h].y = __byte_perm(v.x, v.z, 0x7632);  // (k1, k5)
          xr[i][h].z = __byte_perm(v.y, v.w, 0x5410);  // (k2, k6)
          xr[i][h].w = __byte_perm(v.y, v.w, 0x7632);  // (k3, k7)
        }
      }
    }
    float tot[RES_MAX_SLABS][4];
#pragma unroll
    for (int s = 0; s < RES_MAX_SLABS; ++s) tot[s][0] = tot[s][1] = tot[s][2] = tot[s][3] = 0.f;
    bool ok = true;
#pragma unroll
    for (int s = 0; s < RES_MAX_SLABS; ++s) {
      if (s >= nsl || !ok) continue;
      if (!ptx::mbar_wait_bounded(full_bar(s), 0u, abort_flag, 2, WAIT_NS)) {
        ok = false;
        continue;
      }
      const uint8_t* st = smem + (size_t)s * P.stage_bytes;
      const int n0 = (blockIdx.x + s * gridDim.x) * ROWS;
      const int rows = min(ROWS, N - n0);
      const int rl0 = min(g, rows - 1), rl1 = min(g + 8, rows - 1);
      const uint8_t* w0p = st + (size_t)rl0 * (K / 2) + c * 8;
      const uint8_t* w1p = st + (size_t)rl1 * (K / 2) + c * 8;
      const __nv_bfloat16* sc0 = reinterpret_cast<const __nv_bfloat16*>(st + P.scale_off) + rl0 * P.gpr;
      const __nv_bfloat16* sc1 = reinterpret_cast<const __nv_bfloat16*>(st + P.scale_off) + rl1 * P.gpr;
      const uint8_t* zp0 = st + P.zp_off + rl0 * P.gpr;
      const uint8_t* zp1 = st + P.zp_off + rl1 * P.gpr;
      float acc[4][4] = {};
      int grp = ch_begin / cpg, in_grp = ch_begin - grp * cpg;
      uint32_t zc0 = __byte_perm((uint32_t)zp0[grp], 0x43u, 0x4040), zc1 = __byte_perm((uint32_t)zp1[grp], 0x43u, 0x4040);
#pragma unroll
      for (int i = 0; i < RES_MAX_CPW; ++i) {
        const int ch = ch_begin + i;
        if (ch >= ch_end) break;
        const uint2 wa = *reinterpret_cast<const uint2*>(w0p + ch * 32);
        const uint2 wb = *reinterpret_cast<const uint2*>(w1p + ch * 32);
        const uint32_t wwa[2] = {wa.x, wa.y}, wwb[2] = {wb.x, wb.y};
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const uint32_t a = wwa[w], b = wwb[w];
          const uint32_t a4 = a >> 4, a8 = a >> 8, a12 = a >> 12;
          const uint32_t b4 = b >> 4, b8 = b >> 8, b12 = b >> 12;
          uint32_t a0 = sub_bf16x2((a & 0x000F000Fu) | 0x43004300u, zc0);
          uint32_t a2 = sub_bf16x2((a4 & 0x000F000Fu) | 0x43004300u, zc0);
          uint32_t a1 = sub_bf16x2((b & 0x000F000Fu) | 0x43004300u, zc1);
          uint32_t a3 = sub_bf16x2((b4 & 0x000F000Fu) | 0x43004300u, zc1);
          mma_bf16_16816(acc[2 * w], a0, a1, a2, a3, xr[i][w].x, xr[i][w].y);
          a0 = sub_bf16x2((a8 & 0x000F000Fu) | 0x43004300u, zc0);
          a2 = sub_bf16x2((a12 & 0x000F000Fu) | 0x43004300u, zc0);
          a1 = sub_bf16x2((b8 & 0x000F000Fu) | 0x43004300u, zc1);
          a3 = sub_bf16x2((b12 & 0x000F000Fu) | 0x43004300u, zc1);
          mma_bf16_16816(acc[2 * w + 1], a0, a1, a2, a3, xr[i][w].z, xr[i][w].w);
        }
        if (++in_grp == cpg || ch + 1 == ch_end) {
          const float s0 = __bfloat162float(sc0[grp]), s1 = __bfloat162float(sc1[grp]);
          float sum4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sum4[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
            acc[0][j] = acc[1][j] = acc[2][j] = acc[3][j] = 0.f;
          }
          tot[s][0] = fmaf(sum4[0], s0, tot[s][0]);
          tot[s][1] = fmaf(sum4[1], s0, tot[s][1]);
          tot[s][2] = fmaf(sum4[2], s1, tot[s][2]);
          tot[s][3] = fmaf(sum4[3], s1, tot[s][3]);
          in_grp = 0;
          ++grp;
          if (ch + 1 < ch_end) {
            zc0 = __byte_perm((uint32_t)zp0[grp], 0x43u, 0x4040);
            zc1 = __byte_perm((uint32_t)zp1[grp], 0x43u, 0x4040);
          }
        }
      }
    }
    // ---- combine the K parts of the warps
    float* red = reinterpret_cast<float*>(smem + P.red_off);
    constexpr int PLANE = CWARPS * ROWS * 8;
    auto put = [&](int s, int plane) {
      float* mine = red + (size_t)plane * PLANE + warp * (ROWS * 8);
      mine[g * 8 + 2 * c] = tot[s][0];
      mine[g * 8 + 2 * c + 1] = tot[s][1];
      mine[(g + 8) * 8 + 2 * c] = tot[s][2];
      mine[(g + 8) * 8 + 2 * c + 1] = tot[s][3];
    };
    auto finish = [&](int s, int plane, int e) {   // output e (row, token) of slab s
      const int row = e >> 3, m = e & 7;
      const int n = (blockIdx.x + s * gridDim.x) * ROWS + row;
      if (n < N && m < M) {
        const float* rb = red + (size_t)plane * PLANE + e;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < CWARPS; ++w) v += rb[w * (ROWS * 8)];
        if (bias) v += bias[n];
        y[(size_t)m * N + n] = __ushort_as_bfloat16(f32_to_bf16_bits_ref(v));
      }
    };
    if (red_planes >= nsl) {   // one plane per slab: a single barrier, then all outputs at once
#pragma unroll
      for (int s = 0; s < RES_MAX_SLABS; ++s)
        if (s < nsl) put(s, s);
      asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory");
      if (*abort_flag == 0)
        for (int e = tid; e < nsl * ROWS * 8; e += CWARPS * 32) finish(e / (ROWS * 8), e / (ROWS * 8), e % (ROWS * 8));
    } else {                   // two planes used in turn: one barrier per slab
#pragma unroll
      for (int s = 0; s < RES_MAX_SLABS; ++s) {
        if (s >= nsl) continue;
        put(s, s & 1);
        asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory");
        if (tid < ROWS * 8 && *abort_flag == 0) finish(s, s & 1, tid);
      }
    }
  }
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && status != nullptr) atomicCAS(status, 0, *abort_flag);
}


// ---------------------------------------------------------------------------------------------------------------
// M <= 2: CUDA-core form, weights straight from global memory.  One or two tokens waste 7/8 of every MMA above, and
// mma.sync is the slow legacy tensor path on sm_100, so for these shapes the dot products run as fp32 FMAs.
//
// No shared-memory ring, no producer warp: a lane owns SL fixed 32-k slices of K for the whole kernel and keeps
// their activations in registers (packed bf16, in nibble-pair order); `wpr` warps side by side cover one weight
// row, 16 / wpr row lanes per block walk disjoint contiguous row ranges.  Per row a lane issues one 16-byte
// streaming load per slice (plus the slice's scale and zero point) and keeps PF rows of them in flight, so a block
// of 16 warps has 16 * PF * 512 bytes of weights on their way at any time; nothing in the loop waits on another
// warp.  32 nibbles become 128 + q with the bf16 bit trick and accumulate (128 + q) * x with mixed-precision FMAs
// (bf16 x bf16 + fp32); the zero point comes off as (128 + zp) * sum(x over the slice), then the group scale
// multiplies the fp32 partial sum.  The PF rows of an iteration are reduced together (interleaved warp shuffles);
// with more than one warp per row the partial sums meet in a double-buffered shared array behind one named barrier
// per iteration.
//
// Programmatic dependent launch: every block releases its dependents at once, and when the caller vouches that the
// weights are constant (`early_weights`) the first PF rows are requested BEFORE griddepcontrol.wait, i.e. while the
// previous kernel of the stream is still draining; activations are read and results written only after the wait.
// F16: activations, scales and output are IEEE half instead of bf16; the nibbles become 1024 + q (0x6400 | q).
template <int M_T, int SL, int PF, int MINB, bool F16 = false>
__global__ void __launch_bounds__(512, MINB)
a16_w4_gemv_direct_kernel(const uint16_t* __restrict__ x, const uint8_t* __restrict__ wq,
                          const uint16_t* __restrict__ scale, const uint8_t* __restrict__ zp,
                          const float* __restrict__ bias, uint16_t* __restrict__ y, int N, int K, int group,
                          int wpr, int early_weights) {
  auto to_bits = [](float v) -> uint16_t {
    return F16 ? __half_as_ushort(__float2half_rn(v)) : f32_to_bf16_bits_ref(v);
  };
  __shared__ float red[2][16][PF][M_T];   // [buffer][warp][row of the iteration][token]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = K >> 5;                    // 32-k slices per row
  const int gpr = K / group;
  const int rows_par = 16 / wpr;
  const int rs = warp / wpr, kq = warp - rs * wpr;
  const long long units = (long long)gridDim.x * rows_par;
  const long long unit = (long long)blockIdx.x * rows_par + rs;
  const int r0 = (int)(unit * N / units), r1 = (int)((unit + 1) * N / units);
  const uint16_t* sc16 = scale;
  ptx::griddep_launch_dependents();

  int slice[SL];
  bool live[SL];
  const uint4* wnext[SL];     // the next row to request: rows are requested strictly in order
  const uint16_t* snext[SL];
  const uint8_t* znext[SL];
  const int wstride = K >> 5;  // row pitch in 16-byte units
#pragma unroll
  for (int sl = 0; sl < SL; ++sl) {
    slice[sl] = (sl * wpr + kq) * 32 + lane;
    live[sl] = slice[sl] < T;
    const int sidx = live[sl] ? slice[sl] : 0;
    const size_t gi = (size_t)r0 * gpr + (sidx * 32) / group;
    wnext[sl] = reinterpret_cast<const uint4*>(wq) + (size_t)r0 * wstride + sidx;
    snext[sl] = sc16 + gi;
    znext[sl] = zp + gi;
  }
  uint4 wb[PF][SL];
  uint32_t sb[PF][SL], zb[PF][SL];
#pragma unroll
  for (int p = 0; p < PF; ++p)
#pragma unroll
    for (int sl = 0; sl < SL; ++sl) {
      wb[p][sl] = make_uint4(0u, 0u, 0u, 0u);
      sb[p][sl] = 0u;
      zb[p][sl] = 0u;
    }
  int to_request = r1 - r0;
  auto request = [&](int p) {
    if (to_request > 0) {
#pragma unroll
      for (int sl = 0; sl < SL; ++sl) {
        if (live[sl]) {
          wb[p][sl] = __ldcs(wnext[sl]);
          sb[p][sl] = __ldg(snext[sl]);
          zb[p][sl] = __ldg(znext[sl]);
        }
        wnext[sl] += wstride;
        snext[sl] += gpr;
        znext[sl] += gpr;
      }
    }
    --to_request;
  };
  if (early_weights) {
#pragma unroll
    for (int p = 0; p < PF; ++p) request(p);
  }
  ptx::griddep_wait();
  if (!early_weights) {
#pragma unroll
    for (int p = 0; p < PF; ++p) request(p);
  }

  // this lane's activations as packed bf16 pairs (x_j, x_j+4) per 8 values: the pairing the nibble extraction yields
  uint32_t xw[M_T][SL][16];
  float xsum[M_T][SL];
#pragma unroll
  for (int m = 0; m < M_T; ++m) {
#pragma unroll
    for (int sl = 0; sl < SL; ++sl) {
      xsum[m][sl] = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) xw[m][sl][j] = 0u;
      if (live[sl]) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)slice[sl] * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // 8 bf16 per 16 bytes
          const uint4 v = __ldg(xp + q);
          xw[m][sl][4 * q + 0] = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
          xw[m][sl][4 * q + 1] = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
          xw[m][sl][4 * q + 2] = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
          xw[m][sl][4 * q + 3] = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
          const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (F16) {
              const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&wv[j]));
              xsum[m][sl] += f2.x + f2.y;
            } else {
              xsum[m][sl] += __uint_as_float(wv[j] << 16) + __uint_as_float(wv[j] & 0xffff0000u);
            }
          }
        }
      }
    }
  }

  int it = 0;
  for (int r = r0; r < r1; r += PF, ++it) {
    float part[PF][M_T];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
#pragma unroll
      for (int m = 0; m < M_T; ++m) part[p][m] = 0.f;
      if (r + p < r1) {   // same for every lane of the warp
#pragma unroll
        for (int sl = 0; sl < SL; ++sl) {
          const uint32_t ww[4] = {wb[p][sl].x, wb[p][sl].y, wb[p][sl].z, wb[p][sl].w};
          const float sc = F16 ? __half2float(__ushort_as_half((unsigned short)sb[p][sl])) : __uint_as_float(sb[p][sl] << 16);
          const float zoff = F16 ? 1024.f + (float)zb[p][sl] : __uint_as_float(0x43000000u | (zb[p][sl] << 16));  // 128 + zp, zp <= 127
          float acc[M_T][4];
#pragma unroll
          for (int m = 0; m < M_T; ++m)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[m][q] = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t pq = ((ww[q] >> (4 * j)) & 0x000F000Fu) | (F16 ? 0x64006400u : 0x43004300u);  // {128 + q_j, 128 + q_(j+4)}
#pragma unroll
              for (int m = 0; m < M_T; ++m) {
                if (F16) fma2_f32_f16(acc[m][q], pq, xw[m][sl][4 * q + j]);
                else fma2_f32_bf16(acc[m][q], pq, xw[m][sl][4 * q + j]);
              }
            }
          }
#pragma unroll
          for (int m = 0; m < M_T; ++m) {
            const float raw = (acc[m][0] + acc[m][1]) + (acc[m][2] + acc[m][3]);
            part[p][m] = fmaf(fmaf(-zoff, xsum[m][sl], raw), sc, part[p][m]);  // a dead slice carries sc = 0
          }
        }
        request(p);  // the registers of row r + p are free again: ask for row r + p + PF
      }
    }
    // sum over the 32 lanes.  Four rows at a time fold into one value per lane first (a lane keeps half of its
    // values and hands the other half to its partner), so the 4 rows cost 6 shuffles instead of 20; afterwards lane
    // 8 * i holds row i.
    float mine[M_T];
    int my_row;
    if (PF == 4) {
      const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0;
#pragma unroll
      for (int m = 0; m < M_T; ++m) {
        float k0 = h16 ? part[2 % PF][m] : part[0][m], k1 = h16 ? part[3 % PF][m] : part[1 % PF][m];
        const float s0 = h16 ? part[0][m] : part[2 % PF][m], s1 = h16 ? part[1 % PF][m] : part[3 % PF][m];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
        k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
        float k = h8 ? k1 : k0;
        const float sx = h8 ? k0 : k1;
        k += __shfl_xor_sync(0xffffffffu, sx, 8);
        k += __shfl_xor_sync(0xffffffffu, k, 4);
        k += __shfl_xor_sync(0xffffffffu, k, 2);
        k += __shfl_xor_sync(0xffffffffu, k, 1);
        mine[m] = k;
      }
      my_row = ((lane & 7) == 0) ? (lane >> 3) : -1;
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int p = 0; p < PF; ++p)
#pragma unroll
          for (int m = 0; m < M_T; ++m) part[p][m] += __shfl_xor_sync(0xffffffffu, part[p][m], o);
      my_row = lane < PF ? lane : -1;
#pragma unroll
      for (int m = 0; m < M_T; ++m) {
        mine[m] = 0.f;
#pragma unroll
        for (int p = 0; p < PF; ++p)
          if (p == lane) mine[m] = part[p][m];
      }
    }
    if (wpr == 1) {
      if (my_row >= 0 && r + my_row < r1) {
#pragma unroll
        for (int m = 0; m < M_T; ++m)
          y[(size_t)m * N + r + my_row] = to_bits(bias ? mine[m] + bias[r + my_row] : mine[m]);
      }
    } else {
      if (my_row >= 0) {
#pragma unroll
        for (int m = 0; m < M_T; ++m) red[it & 1][warp][my_row][m] = mine[m];
      }
      // the wpr warps of this row lane run the same number of iterations: one barrier per iteration, and the
      // buffer written two iterations later is read (by warp kq == 0) before that warp reaches the barrier between
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rs), "r"(wpr * 32) : "memory");
      if (kq == 0 && lane < PF * M_T) {
        const int p = lane / M_T, m = lane - p * M_T;
        float v = 0.f;
        for (int w = 0; w < wpr; ++w) v += red[it & 1][warp + w][p][m];
        if (r + p < r1) y[(size_t)m * N + r + p] = to_bits(bias ? v + bias[r + p] : v);
      }
    }
  }
}

}  // namespace

// one or two tokens: fp32 FMAs on the CUDA cores, a lane per 32-k slice (at most 4 slices per lane, 16 warps per row)
// (the activations of a lane live in registers: 16 per slice and token)
static bool gemv_uses_fma(int M, int K, int group) {
  return M <= 2 && K % 32 == 0 && group % 32 == 0 && K <= 32 * 32 * 16 * (M == 1 ? 4 : 2);
}

// In how many ranges of k the ring form runs M tokens: 1 when the activations and two weight stages fit in shared memory;
// else the smallest split (2, 3, 4) of K into equal ranges of whole groups and 64-k chunks that fits (K = 11008: the
// activations of 3 to 8 tokens need two); 0 if none does.
static int gemv_passes(int M, int K, int group) {
  for (int p = 1; p <= 4; ++p) {
    if (K % p != 0) continue;
    const int kl = K / p;
    if (kl % CHUNK_K != 0 || kl % group != 0) continue;
    if (gemv_plan(M, kl, group, true, K).stages >= 2) return p;
  }
  return 0;
}

int a16_w4_gemv_supported(int M, int N, int K, int group, const char** why, bool f16) {
  const char* w = nullptr;
  if (M < 1 || M > MAX_M) w = "M must be in [1, 8]";
  else if (N < 1) w = "empty N";
  else if (group < 1 || K % group != 0) w = "the group size must divide K";
  else if (gemv_uses_fma(M, K, group)) w = nullptr;
  else if (f16) w = "the f16 decode form exists for one or two tokens (K a multiple of 32, at most 65536 / 32768)";
  else if (K % CHUNK_K != 0) w = "K must be a multiple of 64";
  else if (group < CHUNK_K || group % CHUNK_K != 0) w = "group size must be a multiple of 64 dividing K";
  else if (gemv_passes(M, K, group) == 0) w = "two 16-row weight slabs plus the activations do not fit in shared memory";
  if (why) *why = w;
  return w == nullptr;
}

template <int M_T, int SL, int PF, int MINB, bool F16 = false>
static int launch_direct(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                         int N, int K, int group, int wpr, int blocks, int early, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(512);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, a16_w4_gemv_direct_kernel<M_T, SL, PF, MINB, F16>, static_cast<const uint16_t*>(x),
                              static_cast<const uint8_t*>(wq), static_cast<const uint16_t*>(scale),
                              static_cast<const uint8_t*>(zp), bias, static_cast<uint16_t*>(y), N, K, group, wpr,
                              early));
  return B200Q_OK;
}

// Whether two to eight tokens of this shape take the resident form (the block's whole weight slice in shared memory).
int a16_w4_gemv_resident_applies(int N, int K, int group, bool f16) {
  if (f16 || K % CHUNK_K != 0 || group < CHUNK_K || group % CHUNK_K != 0 || K % group != 0) return 0;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return 0;
  const int slabs = (N + ROWS - 1) / ROWS;
  const int blocks = slabs < sms ? slabs : sms;
  const int spb = (slabs + blocks - 1) / blocks;
  const int chunks = K / CHUNK_K;
  if (spb > RES_MAX_SLABS || (chunks + CWARPS - 1) / CWARPS > RES_MAX_CPW) return 0;
  return resident_plan(K, group, spb, 2).total <= 226 * 1024;
}

int a16_w4_gemv_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       int M, int N, int K, int group, int* status, cudaStream_t stream, bool weights_constant, bool f16) {
  const char* why = nullptr;
  if (!a16_w4_gemv_supported(M, N, K, group, &why, f16)) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 gemv: %s", why);
  if ((reinterpret_cast<uintptr_t>(wq) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return set_error(B200Q_ERR_INVALID, "a16 w4 gemv: weights and activations must be 16-byte aligned");
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // two tokens: the tensor-core decode kernel is the faster one where it applies (measured 14.3 us against 16.2 us at
  // N = 11008, K = 4096); the CUDA-core form then only takes what that kernel cannot (groups of 32, K % 64 != 0)
  const bool mma_ok = K % CHUNK_K == 0 && group >= CHUNK_K && group % CHUNK_K == 0 && gemv_passes(M, K, group) > 0;
  {
    // the resident form: the block's whole weight slice in shared memory, activations in registers
    const int slabs = (N + ROWS - 1) / ROWS;
    const int blocks = slabs < sms ? slabs : sms;
    const int spb = (slabs + blocks - 1) / blocks;
    // B200Q_GEMV_RESIDENT (A/B timing): 0 = never, 1 = two to eight tokens (default), 2 = one token too
    static const int resident_mode = [] { const char* v = getenv("B200Q_GEMV_RESIDENT"); return v ? atoi(v) : 1; }();
    if (resident_mode > 0 && (M > 1 || resident_mode > 1) && a16_w4_gemv_resident_applies(N, K, group, f16)) {
      const int planes = resident_plan(K, group, spb, spb).total <= 226 * 1024 ? spb : 2;
      const ResidentPlan RP = resident_plan(K, group, spb, planes);
      if (RP.total <= 226 * 1024) {
        auto rfn = a16_w4_gemv_resident_kernel;
        CUDA_TRY(cudaFuncSetAttribute(rfn, cudaFuncAttributeMaxDynamicSharedMemorySize, RP.total));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = (size_t)RP.total;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        CUDA_TRY(cudaLaunchKernelEx(&cfg, rfn, static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(wq),
                                    static_cast<const __nv_bfloat16*>(scale), static_cast<const uint8_t*>(zp), bias,
                                    static_cast<__nv_bfloat16*>(y), M, N, K, group, spb, planes, weights_constant ? 1 : 0, status));
        return B200Q_OK;
      }
    }
  }
  if (gemv_uses_fma(M, K, group) && (M == 1 || !mma_ok || f16)) {
    // warps per row: the smallest power of two that leaves a lane at most SL slices
    const int T = K / 32;
    const int early = weights_constant ? 1 : 0;
    if (M == 1) {
      int sl = 1, wpr = 1;
      while (wpr < 16 && wpr * 32 < T) wpr *= 2;
      while (sl * wpr * 32 < T) sl *= 2;  // K > 16384: more slices per lane
      const int blocks = 2 * sms;
      if (sl == 1) return f16 ? launch_direct<1, 1, 4, 2, true>(x, wq, scale, zp, bias, y, N, K, group, wpr, blocks, early, stream) : launch_direct<1, 1, 4, 2, false>(x, wq, scale, zp, bias, y, N, K, group, wpr, blocks, early, stream);
      if (sl == 2) return f16 ? launch_direct<1, 2, 4, 1, true>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream) : launch_direct<1, 2, 4, 1, false>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream);
      return f16 ? launch_direct<1, 4, 1, 1, true>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream) : launch_direct<1, 4, 1, 1, false>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream);
    }
    int sl = 1, wpr = 1;
    while (wpr < 16 && wpr * 32 < T) wpr *= 2;
    while (sl * wpr * 32 < T) sl *= 2;
    if (sl == 1) return f16 ? launch_direct<2, 1, 6, 1, true>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream) : launch_direct<2, 1, 6, 1, false>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream);
    return f16 ? launch_direct<2, 2, 3, 1, true>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream) : launch_direct<2, 2, 3, 1, false>(x, wq, scale, zp, bias, y, N, K, group, wpr, sms, early, stream);
  }
  const int passes = gemv_passes(M, K, group);
  if (passes == 0) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 gemv: the weight slabs do not fit in shared memory");
  const int kl = K / passes;
  const GemvPlan P = gemv_plan(M, kl, group, true, K);
  const int slabs = (N + ROWS - 1) / ROWS;
  const int blocks = slabs < sms ? slabs : sms;
  float* ws = nullptr;
  if (passes > 1) {
    // fp32 partial sums [M][N] between the ranges of k: one buffer per (device, stream), launches of a stream run in order
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, DevBuf> scratch;
    std::lock_guard<std::mutex> lock(mu);
    DevBuf& b = scratch[std::make_pair(dev, stream)];
    B200Q_TRY(b.ensure((size_t)MAX_M * N * 4));
    ws = b.as<float>();
  }
  auto kfn = a16_w4_gemv_kernel;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, P.total));
  for (int pass = 0; pass < passes; ++pass) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)P.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int mode = (pass > 0 ? 1 : 0) | (pass + 1 < passes ? 2 : 0);
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(wq),
                                static_cast<const __nv_bfloat16*>(scale), static_cast<const uint8_t*>(zp), bias,
                                static_cast<__nv_bfloat16*>(y), M, N, kl, group, weights_constant ? 1 : 0, status, K, pass * kl, mode,
                                ws));
  }
  return B200Q_OK;
}

}  // namespace b200q

