// A16MatMul with 4-bit group-quantized weights for a handful of tokens (2 <= M <= 32) on the 5th-generation tensor
// cores, built around WARPGROUPS that run without talking to each other.
//
// Semantics: tpu::A16MatMulOp::inference, static w4 path with w_transpose
// (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246): weight bytes [N, K/2], even k in the low nibble,
// W[n,k] = (q - zp[n, k/g]) * scale[n, k/g], y = bf16(x * W^T (+ bias)) with fp32 accumulation.
//
// Why another form.  The pipelined kernel of a16_w4_umma.cu hands 64-k blocks from conversion warps to MMA issuers to
// epilogue warps through mbarriers; for few tokens its time is the latency of those hand-overs, not the work.  Here a
// warpgroup (four warps = the four lane quarters of tensor memory) owns a 128-row tile of one K slice from the first
// byte to the last:
//   * its packed weights arrive by TMA, 128 rows x 128 bytes (256 k) per box with the 128-byte swizzle, two boxes in
//     flight; every lane owns one output channel (TMEM lane = row of the tile) and reads ITS row's 16 bytes (32
//     weights) per step from shared memory - the swizzle makes those reads conflict-free;
//   * the dequantised weight is never rounded: (q - zp) is an exact small integer and scale a 16-bit float, so their
//     product splits exactly into two 16-bit floats, hi = rn(d * s) and lo = fma(d, s, -hi) (the error of a product is
//     representable); both halves go to tensor memory and each K step is two MMAs (hi and lo) into ONE fp32
//     accumulator that lives for the whole slice - no per-group drain, no scale in the epilogue;
//   * the four warps meet at a named barrier (bar.sync, a few cycles) before one of them issues the step's four MMAs;
//     the mbarriers are the TMA's and the one that says a TMEM buffer's MMAs have completed, tested two steps later;
//   * the four warpgroups of a CTA work on four neighbouring tiles of the SAME K slice, so the slice's activations
//     are staged once per CTA as the MMA's B operand (K-major, 128-byte swizzle), in the nibble-pair order
//     0,4,1,5,2,6,3,7 inside every 8 k in which the weights leave the conversion, so no permutes are spent on A;
//   * K slices add up in a float workspace [N][32] with red.global.add.v4.f32, and the warpgroup that arrives last
//     at a tile rounds to the output type, stores y and leaves the workspace zeroed for the next call.
//
// Every wait is bounded; a wait that runs out sets a flag, after which every thread still walks the same loop (without
// work) so that no barrier is left waiting, TMEM is freed and *status receives the code.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

#include "a16.h"
#include "devbuf.h"
#include "igemm.h"
#include "internal.h"
#include "ptx_sm100.cuh"
#include "round16.cuh"

namespace b200q {
namespace {

constexpr int WG_PER_CTA = 4;
constexpr int WG_THREADS = 128;
constexpr int WG_CTA_THREADS = WG_PER_CTA * WG_THREADS;
constexpr int TILE_N = 128;            // output channels per tile = MMA M
constexpr int KSTEP = 32;              // k per step: 16 bytes of nibbles per row, 16 TMEM columns per half
constexpr int CHUNK_STEPS = 8;         // one TMA box: 128 bytes = 256 k per row
constexpr int W_BOX_BYTES = TILE_N * 128;
constexpr int NBUF = 2;                // weight boxes in flight per warpgroup
constexpr int WS_PITCH = 32;           // workspace floats per output channel
constexpr int WG_TMEM_COLS = 128;      // per warpgroup: two A buffers of 32 columns (hi | lo) + the accumulator (<= 64)
constexpr int BARS_PER_WG = NBUF + 3;  // full[NBUF], a_free[2], acc_done
constexpr uint64_t WG_WAIT_NS = 2000000000ull;

struct WgArgs {
  const uint8_t* x;       // 16-bit floats [M][K]
  const uint16_t* scale;  // [N][gpr]
  const uint8_t* zp;      // [N][gpr]
  const float* bias;      // [N] or null
  uint16_t* y;            // [M][N]
  float* ws;              // [N][32] fp32 partial sums, zero between calls
  int* counters;          // [tiles] arrivals per tile, zero between calls
  int M, N, K, group, gpr;
  int tiles;              // ceil(N / 128)
  int tile_groups;        // ceil(tiles / 4): the four warpgroups of a CTA take four neighbouring tiles
  int ksplit;             // K slices
  int kt_per_unit;        // 64-k tiles per slice, even (the last slice may be shorter)
  int num_kt;             // K / 64
  uint32_t idesc;
  int meta_vec;           // 4 / 2: scales and zero points of a chunk are read as one vector each (group 64 / 128); 0: one by one
  int* status;
};

__device__ __forceinline__ void wg_bar(int wg) { asm volatile("bar.sync %0, %1;" ::"r"(wg + 1), "n"(WG_THREADS) : "memory"); }

template <bool F16>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  uint32_t d;
  if (F16) asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
template <bool F16>
__device__ __forceinline__ uint32_t fma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  if (F16) asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// two K = 16 steps (32 k) of A in tensor memory against B in shared memory
__device__ __forceinline__ void umma_2k_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                           uint32_t accumulate_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b32 at, bl;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "setp.eq.b32 p, %4, %4;\n\t"
      "add.u32 at, %1, 8;\n\t"
      "add.u32 bl, %2, 2;\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [at], db, %4, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int NT, bool F16>
__global__ void __launch_bounds__(WG_CTA_THREADS, 1)
a16_w4_wg_kernel(const __grid_constant__ CUtensorMap wmap, const WgArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2, quarter = warp & 3, wtid = threadIdx.x & (WG_THREADS - 1);
  constexpr int B_TILE = NT * 128;                                    // one 64-k tile of activations
  uint8_t* wsm = smem + (size_t)wg * NBUF * W_BOX_BYTES;              // this warpgroup's weight boxes
  uint8_t* bsm = smem + (size_t)WG_PER_CTA * NBUF * W_BOX_BYTES;      // the CTA's activation tiles
  uint8_t* misc = bsm + (size_t)args.kt_per_unit * B_TILE;            // barriers | tmem pointer | abort flag | last flags
  const uint32_t bar0 = ptx::smem_u32(misc) + 8u * (uint32_t)(wg * BARS_PER_WG);
  auto full = [&](int b) { return bar0 + 8u * (uint32_t)b; };
  auto a_free = [&](int b) { return bar0 + 8u * (uint32_t)(NBUF + b); };
  const uint32_t acc_done = bar0 + 8u * (uint32_t)(NBUF + 2);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(misc + 8 * BARS_PER_WG * WG_PER_CTA);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 8 * BARS_PER_WG * WG_PER_CTA + 4);
  volatile int* last_flag = reinterpret_cast<volatile int*>(misc + 8 * BARS_PER_WG * WG_PER_CTA + 8) + wg;

  ptx::griddep_launch_dependents();
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&wmap);
    for (int i = 0; i < BARS_PER_WG * WG_PER_CTA; ++i) ptx::mbar_init(ptx::smem_u32(misc) + 8u * i, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), 512u);
    ptx::tmem_relinquish();
  }
  ptx::griddep_wait();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t_wg = tmem_base + (uint32_t)(wg * WG_TMEM_COLS);                   // columns of this warpgroup
  const uint32_t t_lane = t_wg + ((uint32_t)(quarter * 32) << 16);                  // this warp's lane quarter
  const uint32_t t_acc = t_wg + 64u;
  const uint64_t bdesc0 = ptx::make_smem_desc_kmajor(ptx::smem_u32(bsm), 1024, 2);
  const uint32_t b_hi = (uint32_t)(bdesc0 >> 32), b_lo0 = (uint32_t)bdesc0;
  const uint32_t one2 = F16 ? 0x3C003C00u : 0x3F803F80u;
  const uint32_t magic = F16 ? 0x64006400u : 0x43004300u;
  const int row = quarter * 32 + lane;                                             // row of the tile = TMEM lane
  const uint32_t w_row = ptx::smem_u32(wsm) + (uint32_t)(row * 128);
  const uint32_t w_xor = (uint32_t)(row & 7);

  const int units = args.tile_groups * args.ksplit;
  uint32_t full_phase = 0u;            // bit b: parity of the next completion of full[b]
  uint32_t free_phase[2] = {0u, 0u};   // parity of the next completion to wait for, per A buffer
  uint32_t acc_phase = 0u;
  uint32_t used[2] = {0u, 0u};         // the buffer has MMAs in flight that were never waited for

  auto wait = [&](uint32_t bar, uint32_t parity, int where) {
    if (*abort_flag != 0) return;
    ptx::mbar_wait_bounded_fast<20>(bar, parity, abort_flag, where, WG_WAIT_NS);
  };

  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int tg = u / args.ksplit, slice = u - tg * args.ksplit;
    const int tile = tg * WG_PER_CTA + wg;
    const bool wg_live = tile < args.tiles;
    const int kt0 = slice * args.kt_per_unit;
    const int kts = min(args.kt_per_unit, args.num_kt - kt0);
    const int n = tile * TILE_N + row;
    const bool live = wg_live && n < args.N;
    const int nsteps = kts * 2;
    const int nchunks = (nsteps + CHUNK_STEPS - 1) / CHUNK_STEPS;

    // ---- the first weight boxes (rows past N and bytes past K / 2 arrive as zeros)
    if (wg_live && wtid == 0 && *abort_flag == 0) {
      for (int c = 0; c < NBUF && c < nchunks; ++c) {
        ptx::mbar_arrive_expect_tx(full(c), (uint32_t)W_BOX_BYTES);
        ptx::tma_load_2d(ptx::smem_u32(wsm) + (uint32_t)(c * W_BOX_BYTES), &wmap, full(c), kt0 * 32 + c * 128, tile * TILE_N);
      }
    }
    // ---- scales and zero points of the first chunk (scale in the low half, zero point above it)
    const size_t gbase = (size_t)(live ? n : 0) * args.gpr;
    uint32_t meta_next[CHUNK_STEPS];
    auto load_meta = [&](int c) {
      const int g0 = (kt0 * 64 + c * CHUNK_STEPS * KSTEP) / args.group;
      if (!live) {
#pragma unroll
        for (int e = 0; e < CHUNK_STEPS; ++e) meta_next[e] = 0u;
      } else if (args.meta_vec == 4) {   // 64-k groups: four scales (8 bytes) and four zero points (4 bytes) per chunk
        const uint2 sv = __ldg(reinterpret_cast<const uint2*>(args.scale + gbase + g0));
        const uint32_t zv = __ldg(reinterpret_cast<const uint32_t*>(args.zp + gbase + g0));
        // {scale (16 bits), zero point, unused byte}
        meta_next[0] = meta_next[1] = __byte_perm(sv.x, zv, 0x4410);
        meta_next[2] = meta_next[3] = __byte_perm(sv.x, zv, 0x5532);
        meta_next[4] = meta_next[5] = __byte_perm(sv.y, zv, 0x6610);
        meta_next[6] = meta_next[7] = __byte_perm(sv.y, zv, 0x7732);
      } else if (args.meta_vec == 2) {   // 128-k groups
        const uint32_t sv = __ldg(reinterpret_cast<const uint32_t*>(args.scale + gbase + g0));
        const uint32_t zv = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(args.zp + gbase + g0));
        meta_next[0] = meta_next[1] = meta_next[2] = meta_next[3] = __byte_perm(sv, zv, 0x4410);
        meta_next[4] = meta_next[5] = meta_next[6] = meta_next[7] = __byte_perm(sv, zv, 0x5532);
      } else {
#pragma unroll
        for (int e = 0; e < CHUNK_STEPS; ++e) {
          const int st = c * CHUNK_STEPS + e;
          meta_next[e] = 0u;
          if (st < nsteps) {
            const int gi = (kt0 * 64 + st * KSTEP) / args.group;
            meta_next[e] = (uint32_t)__ldg(args.scale + gbase + gi) | ((uint32_t)__ldg(args.zp + gbase + gi) << 16);
          }
        }
      }
    };
    load_meta(0);

    // ---- the slice's activations into shared memory: [64-k tile][NT rows][128 bytes], 128-byte swizzle, k in pair order
    // (rows >= M are left as they are: row m of B only reaches column m of the accumulator, which nobody reads)
    __syncthreads();   // every warpgroup is done with the previous unit's tiles
    {
      const int total = kts * args.M * 8;
      for (int i0 = threadIdx.x; i0 < total; i0 += 4 * WG_CTA_THREADS) {
        uint4 v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + e * WG_CTA_THREADS;
          if (i < total) {
            const int c = i & 7, r = (i >> 3) % args.M, t = (i >> 3) / args.M;
            v[e] = __ldg(reinterpret_cast<const uint4*>(args.x + ((size_t)r * args.K + (size_t)(kt0 + t) * 64 + c * 8) * 2));
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + e * WG_CTA_THREADS;
          if (i < total) {
            const int c = i & 7, r = (i >> 3) % args.M, t = (i >> 3) / args.M;
            uint4 o;
            o.x = __byte_perm(v[e].x, v[e].z, 0x5410);
            o.y = __byte_perm(v[e].x, v[e].z, 0x7632);
            o.z = __byte_perm(v[e].y, v[e].w, 0x5410);
            o.w = __byte_perm(v[e].y, v[e].w, 0x7632);
            *reinterpret_cast<uint4*>(bsm + (size_t)t * B_TILE + r * 128 + ((c ^ (r & 7)) << 4)) = o;
          }
        }
      }
    }
    ptx::fence_proxy_async_smem();
    __syncthreads();
    if (!wg_live) continue;

    for (int c = 0; c < nchunks; ++c) {
      const int wb = c % NBUF;
      uint32_t meta[CHUNK_STEPS];
#pragma unroll
      for (int e = 0; e < CHUNK_STEPS; ++e) meta[e] = meta_next[e];
      if (c + 1 < nchunks) load_meta(c + 1);
      wait(full(wb), (full_phase >> wb) & 1u, 4);
      full_phase ^= 1u << wb;
      const uint32_t w_box = w_row + (uint32_t)(wb * W_BOX_BYTES);
#pragma unroll
      for (int j = 0; j < CHUNK_STEPS; ++j) {
        const int st = c * CHUNK_STEPS + j;
        if (st >= nsteps) break;
        uint32_t ww[4];
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(ww[0]), "=r"(ww[1]), "=r"(ww[2]), "=r"(ww[3])
                     : "r"(w_box + (((uint32_t)j ^ w_xor) << 4)));
        const uint32_t s2 = __byte_perm(meta[j], 0u, 0x1010);                      // {s, s}
        const uint32_t ns2 = s2 ^ 0x80008000u;
        const uint32_t negz = __byte_perm(meta[j], F16 ? 0xE4u : 0xC3u, 0x4242);    // -(128 + zp) (f16: -(1024 + zp)) twice
        const int b = j & 1;
        if (used[b]) {   // the MMAs that read this buffer two steps ago
          wait(a_free(b), free_phase[b], 1);
          free_phase[b] ^= 1u;
          used[b] = 0u;
          ptx::tc_fence_after_sync();
        }
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t t = ((ww[q] >> (4 * e)) & 0x000F000Fu) | magic;   // {128 + q_e, 128 + q_(e+4)}
            const uint32_t d = fma2<F16>(t, one2, negz);                     // q - zp, exact
            const uint32_t h = mul2<F16>(d, s2);                            // rounded product
            hi[4 * q + e] = h;
            lo[4 * q + e] = fma2<F16>(d, ns2, h);                           // minus its exact remainder (the MMA negates A)
          }
        }
        {
          ptx::tmem_st_32x32b_x16(t_lane + (uint32_t)(b * 32), hi);
          ptx::tmem_st_32x32b_x16(t_lane + (uint32_t)(b * 32 + 16), lo);
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
          wg_bar(wg);
          if (quarter == (j & 3) && lane == 0 && *abort_flag == 0) {   // the issuing role goes round the four warps
            ptx::tc_fence_after_sync();
            const uint32_t bl = b_lo0 + (uint32_t)((st >> 1) * (B_TILE >> 4)) + (uint32_t)((st & 1) * 4);
            umma_2k_ts(t_acc, t_wg + (uint32_t)(b * 32), bl, b_hi, args.idesc, st != 0 ? 1u : 0u);
            umma_2k_ts(t_acc, t_wg + (uint32_t)(b * 32 + 16), bl, b_hi, args.idesc | (1u << 13), 1u);   // bit 13: negate A
            ptx::umma_commit(a_free(b));
            if (st == nsteps - 1) ptx::umma_commit(acc_done);
          }
          used[b] = 1u;
        }
      }
      // every lane has read its rows of this box (the barrier of the chunk's last step): refill it
      if (c + NBUF < nchunks && wtid == 0 && *abort_flag == 0) {
        ptx::mbar_arrive_expect_tx(full(wb), (uint32_t)W_BOX_BYTES);
        ptx::tma_load_2d(ptx::smem_u32(wsm) + (uint32_t)(wb * W_BOX_BYTES), &wmap, full(wb), kt0 * 32 + (c + NBUF) * 128,
                         tile * TILE_N);
      }
    }
    // ---- the slice's sum: into the workspace
    wait(acc_done, acc_phase, 2);
    acc_phase ^= 1u;
    // (the buffers' last commits are covered by acc_done: consume them so that the phases stay in step)
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      if (used[b]) {
        wait(a_free(b), free_phase[b], 3);
        free_phase[b] ^= 1u;
        used[b] = 0u;
      }
    }
    ptx::tc_fence_after_sync();
    const uint32_t t_acc_lane = t_acc + ((uint32_t)(quarter * 32) << 16);
    float* wsrow = args.ws + (size_t)(live ? n : 0) * WS_PITCH;
#pragma unroll
    for (int c0 = 0; c0 < NT; c0 += 16) {
      uint32_t r[16];
      ptx::tmem_ld_32x32b_x16(t_acc_lane + (uint32_t)c0, r);
      ptx::tmem_ld_wait_16(r);
      if (live && *abort_flag == 0) {
#pragma unroll
        for (int c = 0; c < 16; c += 4)
          if (c0 + c < args.M)   // columns past M hold sums of stale shared memory; they are zeroed again by the finisher
            red_add_v4(wsrow + c0 + c, __uint_as_float(r[c]), __uint_as_float(r[c + 1]), __uint_as_float(r[c + 2]),
                       __uint_as_float(r[c + 3]));
      }
    }
    ptx::tc_fence_before_sync();
    // ---- the last warpgroup of a tile finishes it
    __threadfence();
    wg_bar(wg);
    if (wtid == 0) *last_flag = (atomicAdd(args.counters + tile, 1) == args.ksplit - 1) ? 1 : 0;
    wg_bar(wg);
    if (*last_flag != 0) {
      __threadfence();
      if (live) {
        const float bv = args.bias ? args.bias[n] : 0.f;
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 8) {
          if (c0 < args.M) {
            const float4 v0 = __ldcg(reinterpret_cast<const float4*>(wsrow + c0));
            const float4 v1 = __ldcg(reinterpret_cast<const float4*>(wsrow + c0 + 4));
            *reinterpret_cast<float4*>(wsrow + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(wsrow + c0 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (c0 + e < args.M) {
                const float r = v[e] + bv;
                args.y[(size_t)(c0 + e) * args.N + n] = F16 ? __half_as_ushort(__float2half_rn(r)) : f32_to_bf16_bits_ref(r);
              }
            }
          }
        }
      }
      if (wtid == 0) args.counters[tile] = 0;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512u);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && args.status != nullptr) atomicCAS(args.status, 0, *abort_flag);
}

// The float workspace and the tile counters.  A handle brings its own; the stateless entry uses one per (device,
// stream): launches of one stream run in order and each leaves both zeroed, launches of different streams must not
// share them.  Zeroed when (re)allocated.
std::mutex g_wg_mutex;
std::map<std::pair<int, cudaStream_t>, A16WgScratch> g_wg_scratch;

template <int NT, bool F16>
int launch_wg(const CUtensorMap& wmap, WgArgs a, int grid, int smem, cudaStream_t s) {
  a.idesc = ptx::make_idesc(1u, F16 ? 0u : 1u, F16 ? 0u : 1u, (uint32_t)TILE_N, (uint32_t)NT);   // f32 accumulate
  auto kfn = a16_w4_wg_kernel<NT, F16>;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(WG_CTA_THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, wmap, a));
  return B200Q_OK;
}

}  // namespace

int a16_w4_wg_supported(long long M, int N, int K, int group, const char** why) {
  const char* w = nullptr;
  if (M < 1 || M > 32) w = "M must be in [1, 32]";
  else if (N < 1) w = "empty N";
  else if (K % 64 != 0) w = "K must be a multiple of 64";
  else if (group < KSTEP || group % KSTEP != 0 || K % group != 0) w = "the group size must be a multiple of 32 that divides K";
  if (why) *why = w;
  return w == nullptr;
}

int a16_w4_wg_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                     long long M, int N, int K, int group, int* status, cudaStream_t stream, bool f16, A16WgScratch* own) {
  const char* why = nullptr;
  if (!a16_w4_wg_supported(M, N, K, group, &why)) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 warpgroup kernel: %s", why);
  if ((reinterpret_cast<uintptr_t>(wq) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return set_error(B200Q_ERR_INVALID, "a16 w4: weights and activations must be 16-byte aligned");
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int nt = M <= 16 ? 16 : 32;
  WgArgs a{};
  a.x = static_cast<const uint8_t*>(x);
  a.scale = static_cast<const uint16_t*>(scale);
  a.zp = static_cast<const uint8_t*>(zp);
  a.bias = bias;
  a.y = static_cast<uint16_t*>(y);
  a.M = (int)M;
  a.N = N;
  a.K = K;
  a.group = group;
  a.gpr = K / group;
  a.tiles = (N + TILE_N - 1) / TILE_N;
  a.tile_groups = (a.tiles + WG_PER_CTA - 1) / WG_PER_CTA;
  a.num_kt = K / 64;
  a.status = status;
  // K slices: as many as give every SM at most one unit, an even number of 64-k tiles each (a weight box starts on a
  // 16-byte boundary of the row), within the shared memory left for the slice's activations (64 KB)
  const int kt_cap = ((64 * 1024) / (nt * 128)) & ~3;
  int ksplit = sms / a.tile_groups;
  if (ksplit < 1) ksplit = 1;
  int kt_per = (a.num_kt + ksplit - 1) / ksplit;
  kt_per = (kt_per + 3) & ~3;   // whole chunks: a chunk's scales and zero points then start on a vector boundary
  if (kt_per > kt_cap) kt_per = kt_cap;
  ksplit = (a.num_kt + kt_per - 1) / kt_per;
  a.ksplit = ksplit;
  a.kt_per_unit = kt_per;
  {
    const int gpc = (CHUNK_STEPS * KSTEP) / group;   // groups per chunk
    const bool aligned = (reinterpret_cast<uintptr_t>(scale) & 7) == 0 && (reinterpret_cast<uintptr_t>(zp) & 3) == 0;
    a.meta_vec = ((gpc == 4 || gpc == 2) && aligned && a.gpr % gpc == 0) ? gpc : 0;
  }
  const long long units = (long long)a.tile_groups * ksplit;
  const int grid = (int)(units < sms ? units : sms);
  const int smem = WG_PER_CTA * NBUF * W_BOX_BYTES + kt_per * nt * 128 + 8 * BARS_PER_WG * WG_PER_CTA + 8 + 4 * WG_PER_CTA + 1024 + 64;

  CUtensorMap wmap;
  {
    const uint64_t dims[2] = {(uint64_t)(K / 2), (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)(K / 2)};
    const uint32_t box[2] = {128u, (uint32_t)TILE_N};
    B200Q_TRY(make_tmap_u8(&wmap, wq, 2, dims, strides, box));
  }

  std::lock_guard<std::mutex> lock(g_wg_mutex);
  A16WgScratch& sc = own ? *own : g_wg_scratch[std::make_pair(dev, stream)];
  const size_t need = (size_t)a.tiles * TILE_N * WS_PITCH;
  if (need > sc.ws_elems) {
    B200Q_TRY(sc.ws.ensure(need * 4));
    CUDA_TRY(cudaMemsetAsync(sc.ws.p, 0, need * 4, stream));
    sc.ws_elems = need;
  }
  if (a.tiles > sc.tiles) {
    B200Q_TRY(sc.counters.ensure((size_t)a.tiles * 4));
    CUDA_TRY(cudaMemsetAsync(sc.counters.p, 0, (size_t)a.tiles * 4, stream));
    sc.tiles = a.tiles;
  }
  a.ws = static_cast<float*>(sc.ws.p);
  a.counters = static_cast<int*>(sc.counters.p);
  if (f16) return nt == 16 ? launch_wg<16, true>(wmap, a, grid, smem, stream) : launch_wg<32, true>(wmap, a, grid, smem, stream);
  return nt == 16 ? launch_wg<16, false>(wmap, a, grid, smem, stream) : launch_wg<32, false>(wmap, a, grid, smem, stream);
}

}  // namespace b200q
