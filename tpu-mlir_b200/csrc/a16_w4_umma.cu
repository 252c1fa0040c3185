// A16MatMul with 4-bit group-quantized weights on the 5th-generation tensor cores: the packed weights are dequantised
// in registers and handed to tcgen05.mma as its A operand through TENSOR MEMORY (kind::f16, bf16 x bf16, fp32
// accumulation in TMEM); they never exist in global or shared memory in any wider form.
//
// Semantics: tpu::A16MatMulOp::inference, static w4 path with w_transpose
// (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246): weight bytes [N, K/2], even k in the low
// nibble, W[n,k] = (q - zp[n, k/g]) * scale[n, k/g], y = bf16(x * W^T (+ bias)) with fp32 accumulation.  The
// reference keeps W in fp32 (A16MatMul.cpp:190-198 does not round it); so does this kernel in effect: the tensor
// cores multiply the exact small integers (q - zp) with the bf16 activations, and the group scale multiplies the
// fp32 partial sum of each group afterwards.
//
// The product is computed transposed, D[n, m] = sum_k A[n, k] * B[m, k]: the 128 TMEM lanes are output channels,
// the columns are tokens.  One persistent CTA per SM, 32 warps:
//   warp 0        TMA producer of the packed weights: boxes of 16 rows x 128 bytes (= 256 k, four k-blocks) with the
//                 128-byte swizzle into a ring of raw stages.
//   warp 1        owns TMEM, issues the MMAs (one thread): per k-block of 64 k four MMAs 128 x N x 16, A from TMEM.
//   warp 2        many-token form: TMA producer of the activation tile (B operand) of each k-block.
//   dequantisers  W warps per TMEM lane quarter.  The warp of quarter q with slot s converts its quarter's 32 rows of
//                 every k-block j with j mod W == s: a lane reads its row's 32 bytes of nibbles, turns each 32-bit word
//                 into 128 + q as bf16 by the bit trick, subtracts (128 + zp) with one packed bf16 FMA, and writes the
//                 64 values as 32 columns of its TMEM lane (tcgen05.st).  A k-block is complete when the four
//                 quarters have arrived on its barrier.
//   epilogue      drains the accumulator of each period, running[n][m] += scale[n][g] * partial; at the end of a
//                 work item adds the bias, rounds to bf16 and stores y[m][n].
//
// Groups and columns.  The group scale cannot ride through the MMA, so partial sums of different groups must stay
// apart.  With many tokens the accumulator is drained after every group (several TMEM buffers alternate).  With few
// tokens (M <= 4) the accumulator has spare columns: column j = g_local * MTOK + m belongs to group g_local of the
// current period of G = 16 / MTOK groups, and the B operand of a k-block of group g_local is zero except in its MTOK
// rows.  That operand is a window into one small buffer, (G-1)*MTOK zero rows | the MTOK activation rows | (G-1)*MTOK
// zero rows, starting (G-1-g_local)*MTOK rows into it, so only the MTOK live rows are rewritten per k-block (from a copy
// of the activations that stays in shared memory).  One drain then serves G groups: for one token and K = 4096, four
// drains per row instead of 64.
//
// Rows and lanes.  A work item covers up to 128 output channels; with few tokens the items are smaller (a multiple of
// 16 rows) so that every SM gets one.  Row r of an item lives in TMEM lane 32 * q + 8 * (r / 32) + r % 8 with
// q = (r / 8) % 4: 8-row groups go round the four lane quarters, so a partial item still loads the quarters evenly.
//
// Every mbarrier wait is bounded (2 s); a wait that runs out leaves its site code in a shared flag, every role
// unwinds, TMEM is freed and *status receives the code.
#include <cuda.h>

#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "a16.h"
#include "igemm.h"
#include "internal.h"
#include "ptx_sm100.cuh"
#include "round16.cuh"

namespace b200q {
namespace {

constexpr int TILE_ROWS = 128;           // output channels per work item = MMA M
constexpr int KB = 64;                   // k per k-block: 64 bf16 = one 128-byte swizzle span of B
constexpr int RAW_KB = 4;                // k-blocks per raw stage (128 bytes of nibbles per row)
constexpr int RAW_STAGE_BYTES = TILE_ROWS * 128;
constexpr int A_COLS = 32;               // TMEM columns of one k-block of A (two bf16 per column)
constexpr int TMEM_COLS = 512;
constexpr int MAX_RAW = 8, MAX_AS = 12, MAX_ACC = 8;
constexpr int THREADS = 1024;
constexpr int SCALE_PITCH = TILE_ROWS + 2;   // scaleT[g][n], bf16: transposed so that lanes (rows) read one group conflict-free
constexpr int ZP_PITCH = TILE_ROWS + 4;      // zpT[g][n], bytes
constexpr uint64_t WAIT_NS = 2000000000ull;
#ifndef POLL_SLEEP_NS
#define POLL_SLEEP_NS 300
#endif

// MT == 0: few-token form (M <= 4); else the token tile width of the many-token form
template <int MT>
struct Cfg {
  static constexpr bool FEW = MT == 0;
  // MMA-issuing threads.  One thread issuing every k-block's four MMAs, two commits and two barrier tests is the
  // slowest actor of the kernel for narrow token tiles (each of those instructions takes it 50-100 cycles), so the
  // drain periods go round NI issuers (lane 0 of warps 0..NI-1, one per scheduler): period P runs on issuer P % NI
  // into accumulator P % NACC, and an accumulator always belongs to the same issuer (NI divides NACC).
  static constexpr int NI = (FEW || MT == 128) ? 1 : 4;
  static constexpr int RAW_WARP = NI > 1 ? 4 : 0, B_WARP = NI > 1 ? 5 : 2;   // the two TMA producers
  static constexpr int W = FEW ? 6 : (MT == 128 ? 3 : 4);     // dequantisation warps per lane quarter
  static constexpr int E = FEW ? 4 : (MT == 128 ? 16 : 8);    // epilogue warps (a multiple of 4)
  static constexpr int N_MMA = FEW ? 16 : MT;
  static constexpr int NACC = FEW ? 2 : (MT == 128 ? 2 : 4);  // accumulator buffers
  // accumulators are handed over in sets: the MMA thread signals a set when its last group is complete and the epilogue
  // drains the whole set behind ONE wait / arrive pair (the hand-over, not the arithmetic, is what a drain costs)
#ifndef UMMA_SET_DIV
#define UMMA_SET_DIV 2
#endif
  static constexpr int SET = (FEW || NI > 1) ? 1 : (NACC / UMMA_SET_DIV > 0 ? NACC / UMMA_SET_DIV : 1);
  static_assert(NACC % NI == 0, "an accumulator belongs to one issuer");
  static constexpr int AS = FEW ? 12 : (MT == 32 ? 12 : 8);   // k-blocks of A in TMEM (what is in flight between conversion and MMA)
  static constexpr int A_COL0 = TMEM_COLS - AS * A_COLS;      // accumulators from column 0, A stages at the top
  static constexpr int B_STAGE_BYTES = FEW ? 32 * 128 : MT * 128;
  static constexpr int FIRST_DQ = NI > 1 ? 8 : 4, FIRST_EPI = FIRST_DQ + 4 * W;
  static constexpr int MY_COLS = N_MMA / (E / 4);             // accumulator columns per epilogue thread
  static_assert(FIRST_EPI + E == THREADS / 32, "32 warps");
  static_assert(NACC * N_MMA <= A_COL0, "accumulators and A stages share 512 columns");
  // shared memory: raw ring | B ring | barriers | misc | scaleT | zpT | resident activations (few-token form)
  static constexpr int NUM_BARS = 2 * MAX_RAW + 2 * MAX_AS + 2 * MAX_ACC + 2;
  __host__ __device__ static int b_off(int rs) { return rs * RAW_STAGE_BYTES; }
  __host__ __device__ static int bar_off(int rs) { return b_off(rs) + AS * B_STAGE_BYTES; }
  __host__ __device__ static int misc_off(int rs) { return bar_off(rs) + NUM_BARS * 8; }
  __host__ __device__ static int meta_off(int rs) { return (misc_off(rs) + 16 + 127) & ~127; }
  __host__ __device__ static int x_off(int rs, int gpr) { return meta_off(rs) + ((gpr * (SCALE_PITCH * 2 + ZP_PITCH) + 15) & ~15); }
  __host__ __device__ static int total(int rs, int gpr, int x_bytes) { return x_off(rs, gpr) + x_bytes + 1024; }
};

struct UmmaArgs {
  const uint8_t* x;       // bf16 [M][K]
  const uint16_t* scale;  // bf16 [N][gpr]
  const uint8_t* zp;      // u8 [N][gpr]
  const float* bias;      // [N] or null
  uint16_t* y;            // bf16 [M][N]
  int M, N, K, group, gpr;
  int num_kb;             // K / 64
  int kpg;                // k-blocks per group
  int mtok;               // few-token form: token rows per group slot (1, 2 or 4)
  int G;                  // groups per drain period
  int rows_item;          // output channels per work item (multiple of 16, <= 128)
  int items_n, items_m;   // work items: items_n row chunks x items_m token tiles
  int ni;                 // MMA issuers in use (1, 2 or 4): chosen so that a stage of A is always consumed by the same issuer
  int raw_box_rows;       // rows of one raw-weight TMA box: rows_item (one box per raw stage) or 16
  int raw_stages;         // depth of the raw ring (chosen by the host so that everything fits in shared memory)
  uint32_t idesc;
  int* status;
  int debug;   // timing experiments only (B200Q_UMMA_DEBUG), bits: 1 = conversion warps skip the arithmetic and the TMEM stores, 2 = no MMAs are issued
};

// 8 nibbles of `w` (k0..k7, k0 lowest) -> four packed 16-bit float words {q_j - zp, q_(j+4) - zp}, j = 0..3.
// bf16: 0x4300 | q = 128 + q (ulp 1 at 128..255); f16: 0x6400 | q = 1024 + q (ulp 1 at 1024..2047).
template <bool F16 = false>
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t negz, uint32_t (&p)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | (F16 ? 0x64006400u : 0x43004300u);
    if (F16) asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(p[j]) : "r"(t), "r"(0x3C003C00u), "r"(negz));  // exact: small integers
    else asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(p[j]) : "r"(t), "r"(0x3F803F80u), "r"(negz));
  }
}
// the 16-bit storage type of activations, scales and output
template <bool F16>
__device__ __forceinline__ float bits_to_f32(uint32_t b) {
  return F16 ? __half2float(__ushort_as_half((unsigned short)b)) : __uint_as_float(b << 16);
}
template <bool F16>
__device__ __forceinline__ uint16_t f32_to_bits(float v) {
  return F16 ? __half_as_ushort(__float2half_rn(v)) : f32_to_bf16_bits_ref(v);
}

// Scales (bf16) or zero points (bytes) of the rows [row0, row0 + nrows) transposed into shared memory as T[g][n]:
// every thread first requests all its 16-byte pieces, then scatters them (one round trip to global memory).
template <typename T, int PITCH>
__device__ __forceinline__ void stage_meta(T* dstT, const T* src, int row0, int nrows, int gpr, int tid, int nthreads) {
  constexpr int PER = 16 / (int)sizeof(T);   // entries per 16-byte piece
  const T* base = src + (size_t)row0 * gpr;
  const int total = nrows * gpr;
  if ((gpr % PER) == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
    const int pieces = total / PER;
    constexpr int BATCH = 4;
    for (int p0 = tid; p0 < pieces; p0 += nthreads * BATCH) {
      uint4 v[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int p = p0 + u * nthreads;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (p < pieces) v[u] = __ldg(reinterpret_cast<const uint4*>(base) + p);
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int p = p0 + u * nthreads;
        if (p < pieces) {
          const int i = p * PER, n = i / gpr, g = i - n * gpr;
          const uint32_t wv[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int k = 0; k < PER; ++k) {
            const uint32_t word = wv[(k * (int)sizeof(T)) >> 2];
            dstT[(g + k) * PITCH + n] = (T)(word >> (8 * ((k * (int)sizeof(T)) & 3)));
          }
        }
      }
    }
  } else {
    constexpr int BATCH = 8;
    for (int i0 = tid; i0 < total; i0 += nthreads * BATCH) {
      T v[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = i0 + u * nthreads;
        v[u] = i < total ? __ldg(base + i) : T(0);
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = i0 + u * nthreads;
        if (i < total) {
          const int n = i / gpr, g = i - n * gpr;
          dstT[g * PITCH + n] = v[u];
        }
      }
    }
  }
}

template <int MT, bool F16 = false>
__global__ void __launch_bounds__(THREADS, 1)
a16_w4_umma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const UmmaArgs args) {
  using C = Cfg<MT>;
  constexpr bool FEW = C::FEW;
  constexpr int W = C::W, E = C::E, AS = C::AS, NACC = C::NACC, N_MMA = C::N_MMA, SET = C::SET, NSETS = NACC / SET;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int RS = args.raw_stages;
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int b_off = C::b_off(RS), misc_off = C::misc_off(RS), meta_off = C::meta_off(RS);
  const uint32_t bar_base = smem_base + (uint32_t)C::bar_off(RS);
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto raw_empty = [&](int s) { return bar_base + 8u * (MAX_RAW + s); };
  auto a_full = [&](int s) { return bar_base + 8u * (2 * MAX_RAW + s); };
  auto a_empty = [&](int s) { return bar_base + 8u * (2 * MAX_RAW + MAX_AS + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * MAX_RAW + 2 * MAX_AS + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * MAX_RAW + 2 * MAX_AS + MAX_ACC + a); };
  const uint32_t dq_sync_bar = bar_base + 8u * (2 * MAX_RAW + 2 * MAX_AS + 2 * MAX_ACC), epi_sync_bar = dq_sync_bar + 8u;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);
  uint16_t* scaleT = reinterpret_cast<uint16_t*>(smem + meta_off);
  uint8_t* zpT = smem + meta_off + args.gpr * SCALE_PITCH * 2;
  // few-token form: the activations, resident for the whole kernel: xs[m][K] bf16, each 16-byte piece already in the
  // nibble-pair order of the A operand
  uint8_t* xs = smem + C::x_off(RS, args.gpr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Meeting point of the warps of a role on an mbarrier (one arrival per warp), with the same bounded wait as every
  // other wait of the kernel: a plain bar.sync would hang if one warp had already given up.
  auto role_sync = [&](uint32_t bar, uint32_t& count, int where) -> bool {
    __syncwarp();
    bool ok_ = true;
    if (lane == 0) {
      ptx::mbar_arrive(bar);
      ok_ = ptx::mbar_wait_bounded_fast(bar, count & 1u, abort_flag, where, WAIT_NS);
    }
    ++count;
    ok_ = __shfl_sync(0xffffffffu, ok_, 0);
    return ok_;
  };
  // every lane of the warp runs the same wait (the barrier test is one warp instruction either way)
  // (the conversion and epilogue warps have slack: they sleep longer between polls so that the single MMA-issuing
  // thread, which shares a scheduler with eight of them, gets the issue slots)
  auto warp_wait = [&](uint32_t bar, uint32_t parity, int where) -> bool {
    return ptx::mbar_wait_bounded_fast<POLL_SLEEP_NS>(bar, parity, abort_flag, where, WAIT_NS);
  };

  ptx::griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      ptx::mbar_init(raw_full(s), 1);
      ptx::mbar_init(raw_empty(s), 4 * RAW_KB);   // one arrival per (k-block, lane quarter)
    }
    for (int s = 0; s < AS; ++s) {
      ptx::mbar_init(a_full(s), FEW ? 4 : 5);     // the four quarters (+ the activation tile's TMA)
      ptx::mbar_init(a_empty(s), 1);
    }
    for (int a = 0; a < NSETS; ++a) {   // one pair of barriers per SET of accumulators
      ptx::mbar_init(acc_full(a), 1);
      ptx::mbar_init(acc_empty(a), E);
    }
    ptx::mbar_init(dq_sync_bar, 4 * W);
    ptx::mbar_init(epi_sync_bar, E);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_w);
    if (!FEW) ptx::prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), (uint32_t)TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::griddep_wait();
  if (FEW) {
    // the window buffers start as zeros; only their live rows are ever rewritten
    uint4* b = reinterpret_cast<uint4*>(smem + b_off);
    for (int i = threadIdx.x; i < AS * C::B_STAGE_BYTES / 16; i += THREADS) b[i] = make_uint4(0u, 0u, 0u, 0u);
    // activations: rows past M are zeros
    const int pieces = args.mtok * (args.K >> 3);
    for (int i = threadIdx.x; i < pieces; i += THREADS) {
      const int m = i / (args.K >> 3), c = i - m * (args.K >> 3);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < args.M) v = __ldg(reinterpret_cast<const uint4*>(args.x + ((size_t)m * args.K + (size_t)c * 8) * 2));
      uint4 o;   // k order 0,4,1,5,2,6,3,7
      o.x = __byte_perm(v.x, v.z, 0x5410);
      o.y = __byte_perm(v.x, v.z, 0x7632);
      o.z = __byte_perm(v.y, v.w, 0x5410);
      o.w = __byte_perm(v.y, v.w, 0x7632);
      reinterpret_cast<uint4*>(xs)[i] = o;
    }
    ptx::fence_proxy_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // work items of this CTA: a contiguous range, token tiles innermost (consecutive items share their weight rows'
  // scales and zero points).  Every role walks the same sequence of k-blocks, raw stages and drain periods; ring
  // positions derive from running counts: k-block j of the CTA uses A stage j % AS in phase (j / AS) & 1.
  const int items = args.items_n * args.items_m;
  const int item_begin = (int)((long long)blockIdx.x * items / gridDim.x);
  const int item_end = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);
  const int num_kb = args.num_kb;
  const int raws_per_item = (num_kb + RAW_KB - 1) / RAW_KB;
  const int kb_per_period = args.G * args.kpg;
  const int periods_per_item = (num_kb + kb_per_period - 1) / kb_per_period;

  if (warp == C::RAW_WARP) {
    // ------------------------------------------------------------ TMA producer: packed weights
    if (lane == 0) {
      bool ok = true;
      int rs = 0;
      uint32_t rphase = 0;
      for (int it = item_begin; it < item_end && ok; ++it) {
        const int in_ = it / args.items_m;
        const int row0 = in_ * args.rows_item;
        const int nrows = min(args.rows_item, args.N - row0);
        // one box of rows_item rows per raw stage where the tensor map was built that way (rows past N arrive as
        // zeros and count), else 16-row boxes
        const int brows = args.raw_box_rows;
        const int boxes = (nrows + brows - 1) / brows;
        for (int rsi = 0; rsi < raws_per_item; ++rsi) {
          ok = ptx::mbar_wait_bounded_fast(raw_empty(rs), rphase ^ 1u, abort_flag, 1, WAIT_NS);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(raw_full(rs), (uint32_t)(boxes * brows) * 128u);
          const uint32_t dst = smem_base + (uint32_t)rs * RAW_STAGE_BYTES;
          for (int b = 0; b < boxes; ++b) ptx::tma_load_2d(dst + (uint32_t)(b * brows) * 128u, &tmap_w, raw_full(rs), rsi * 128, row0 + b * brows);
          // a last raw stage with fewer than four k-blocks: nobody reads the missing ones, stand in for their arrivals
          const int nreal = min(RAW_KB, num_kb - rsi * RAW_KB);
          if (nreal < RAW_KB) ptx::mbar_arrive_n(raw_empty(rs), (uint32_t)(4 * (RAW_KB - nreal)));
          if (++rs == RS) {
            rs = 0;
            rphase ^= 1u;
          }
        }
      }
    }
  } else if (warp == C::B_WARP) {
    // ------------------------------------------------------------ TMA producer: activation tiles (many-token form)
    if (!FEW && lane == 0) {
      bool ok = true;
      int as = 0;
      uint32_t aphase = 0;
      for (int it = item_begin; it < item_end && ok; ++it) {
        const int im = it % args.items_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait_bounded_fast(a_empty(as), aphase ^ 1u, abort_flag, 2, WAIT_NS);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(a_full(as), (uint32_t)C::B_STAGE_BYTES);
          ptx::tma_load_2d(smem_base + (uint32_t)b_off + (uint32_t)as * C::B_STAGE_BYTES, &tmap_x, a_full(as), kb * 128, im * MT);
          if (++as == AS) {
            as = 0;
            aphase ^= 1u;
          }
        }
      }
    }
  } else if (C::NI > 1 && warp < C::NI) {
    // ------------------------------------------------------------ MMA issuers (one per scheduler)
    if (lane == 0) {
      bool ok = true;
      const uint64_t bdesc0 = ptx::make_smem_desc_kmajor(smem_base + (uint32_t)b_off, 1024, 2);
      const uint32_t b_hi = (uint32_t)(bdesc0 >> 32);
      const uint32_t b_lo0 = (uint32_t)bdesc0;
      const uint32_t a_t0 = tmem_base + (uint32_t)C::A_COL0;
      const uint32_t idesc = args.idesc;
      // An mbarrier tells only the parity of its phase, so the issuer that waits for the n-th filling of a stage must
      // be the one that consumed the (n-1)-th (else it could take the completion of filling n-2 for the one it needs):
      // the host picks the number of issuers in use so that a stage always meets the same issuer.
      const int NI = args.ni;
      for (int it = item_begin; it < item_end && ok && warp < NI; ++it) {
        const int pbase = (it - item_begin) * periods_per_item, jbase = (it - item_begin) * num_kb;
        int p = (warp - pbase % NI + NI) % NI;   // this issuer's first period of the item
        for (; p < periods_per_item && ok; p += NI) {
          const int P = pbase + p, acc = P % NACC;
          ok = ptx::mbar_wait_bounded_fast(acc_empty(acc), (((uint32_t)(P / NACC)) & 1u) ^ 1u, abort_flag, 3, WAIT_NS);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const int kb0 = p * kb_per_period, kb1 = min(kb0 + kb_per_period, num_kb);
          for (int kb = kb0; kb < kb1; ++kb) {
            const int j = jbase + kb, as = j % AS;
            ok = ptx::mbar_wait_bounded_fast(a_full(as), ((uint32_t)(j / AS)) & 1u, abort_flag, 4, WAIT_NS);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            if (!(args.debug & 2))
              ptx::umma_kblock_f16_ts(tmem_base + (uint32_t)(acc * N_MMA), a_t0 + (uint32_t)(as * A_COLS),
                                      b_lo0 + (uint32_t)as * (uint32_t)(C::B_STAGE_BYTES >> 4), b_hi, idesc, kb != kb0 ? 1u : 0u);
            ptx::umma_commit(a_empty(as));
          }
          if (!ok) break;
          ptx::umma_commit(acc_full(acc));
        }
      }
    }
  } else if (C::NI == 1 && warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      const uint64_t bdesc0 = ptx::make_smem_desc_kmajor(smem_base + (uint32_t)b_off, 1024, 2);
      const uint32_t b_hi = (uint32_t)(bdesc0 >> 32);
      const uint32_t b_lo0 = (uint32_t)bdesc0;
      const uint32_t a_t0 = tmem_base + (uint32_t)C::A_COL0;
      const uint32_t idesc = args.idesc;
      const int kpg = args.kpg;
      // few-token form: the window of group slot g starts (G - 1 - g) * mtok rows (of 128 bytes) into the buffer
      const uint32_t b_row_step = FEW ? (uint32_t)args.mtok * 8u : 0u;
      const uint32_t b_row_first = FEW ? (uint32_t)(args.G - 1) * b_row_step : 0u;
      int as = 0, acc = 0;
      uint32_t aphase = 0, acc_phase = 0;
      uint32_t a_t = a_t0, b_lo = b_lo0;
      for (int it = item_begin; it < item_end && ok; ++it) {
        int in_period = 0, in_group = 0;
        uint32_t b_row = b_row_first;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (in_period == 0 && acc % SET == 0) {   // the first accumulator of a set: the epilogue has drained the set
            ok = ptx::mbar_wait_bounded_fast(acc_empty(acc / SET), acc_phase ^ 1u, abort_flag, 3, WAIT_NS);
            if (!ok) break;
            ptx::tc_fence_after_sync();
          }
          ok = ptx::mbar_wait_bounded_fast(a_full(as), aphase, abort_flag, 4, WAIT_NS);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          if (!(args.debug & 2)) ptx::umma_kblock_f16_ts(tmem_base + (uint32_t)(acc * N_MMA), a_t, b_lo + b_row, b_hi, idesc, in_period != 0 ? 1u : 0u);
          ptx::umma_commit(a_empty(as));
          if (++as == AS) {
            as = 0;
            aphase ^= 1u;
            a_t = a_t0;
            b_lo = b_lo0;
          } else {
            a_t += A_COLS;
            b_lo += C::B_STAGE_BYTES >> 4;
          }
          if (++in_group == kpg) {
            in_group = 0;
            b_row -= b_row_step;
          }
          if (++in_period == kb_per_period || kb == num_kb - 1) {
            in_period = 0;
            b_row = b_row_first;
            const bool item_done = kb == num_kb - 1;
            if ((acc + 1) % SET == 0 || item_done) {
              ptx::umma_commit(acc_full(acc / SET));          // the set (or what the item fills of it) is complete
              acc = (acc / SET + 1) * SET;                     // an item always starts on a set boundary
            } else {
              ++acc;
            }
            if (acc == NACC) {
              acc = 0;
              acc_phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp >= C::FIRST_DQ && warp < C::FIRST_EPI) {
    // ------------------------------------------------------------ dequantisation warps
    const int dq = warp - C::FIRST_DQ;
    const int quarter = warp & 3;                 // the TMEM lane quarter this warp may write (FIRST_DQ is a multiple of 4)
    const int slot = dq >> 2;                     // 0..W-1
    const int dtid = dq * 32 + lane;
    const int row = 8 * (4 * (lane >> 3) + quarter) + (lane & 7);   // row of the work item held by this TMEM lane
    bool ok = true;
    int staged_chunk = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int live_row0 = (args.G - 1) * mtok;    // few-token form: first live row of the window buffer
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)C::A_COL0;
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int in_ = it / args.items_m;
      const int row0 = in_ * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      if (in_ != staged_chunk) {
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;  // everyone is done with the previous chunk's
        stage_meta<uint8_t, ZP_PITCH>(zpT, args.zp, row0, nrows, args.gpr, dtid, 4 * W * 32);
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;
        staged_chunk = in_;
      }
      const bool live = row < nrows;
      const int jbase = (it - item_begin) * num_kb, rbase = (it - item_begin) * raws_per_item;
      int kb = slot - jbase % W;
      if (kb < 0) kb += W;
      for (; kb < num_kb; kb += W) {
        const int j = jbase + kb, as = j % AS;
        const uint32_t aphase = (uint32_t)(j / AS) & 1u;
        const int r = rbase + kb / RAW_KB, rs = r % RS, sub = kb & (RAW_KB - 1);
        if (!(ok = warp_wait(raw_full(rs), (uint32_t)(r / RS) & 1u, 6))) break;
        // this lane's row: 32 bytes of nibbles = logical 16-byte chunks 2*sub and 2*sub+1 of the swizzled raw row
        uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = w0;
        if (live) {
          const uint8_t* rrow = smem + (size_t)rs * RAW_STAGE_BYTES + row * 128;
          w0 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub) ^ (row & 7)) << 4));
          w1 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub + 1) ^ (row & 7)) << 4));
        }
        const uint32_t z = live ? zpT[(kb / args.kpg) * ZP_PITCH + row] : 0u;
        const uint32_t negz = __byte_perm(z, F16 ? 0xE4u : 0xC3u, 0x4040);  // {-(128 + zp)} x2 as bf16: 0xC300 | zp; f16 -(1024 + zp): 0xE400 | zp
        if (!(ok = warp_wait(a_empty(as), aphase ^ 1u, 7))) break;
        ptx::tc_fence_after_sync();
        const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int h = 0; h < 2 && !(args.debug & 1); ++h) {
          uint32_t o[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t p[4];
            dequant_word<F16>(ww[4 * h + q], negz, p);
            if (FEW) {   // k order 0,4,1,5,2,6,3,7 inside every 8 (B is written in the same order)
              o[4 * q + 0] = p[0];
              o[4 * q + 1] = p[1];
              o[4 * q + 2] = p[2];
              o[4 * q + 3] = p[3];
            } else {     // natural k order: B arrives by TMA
              o[4 * q + 0] = __byte_perm(p[0], p[1], 0x5410);
              o[4 * q + 1] = __byte_perm(p[2], p[3], 0x5410);
              o[4 * q + 2] = __byte_perm(p[0], p[1], 0x7632);
              o[4 * q + 3] = __byte_perm(p[2], p[3], 0x7632);
            }
          }
          ptx::tmem_st_32x32b_x16(t_lane + (uint32_t)(as * A_COLS + 16 * h), o);
        }
        if (FEW && quarter == 0) {
          // this k-block's activations from the resident copy into the live rows of the window buffer
          uint8_t* bst = smem + b_off + (size_t)as * C::B_STAGE_BYTES;
          if (lane < mtok * 8) {
            const int m = lane >> 3, ch = lane & 7, rr = live_row0 + m;
            const uint4 v = *reinterpret_cast<const uint4*>(xs + ((size_t)m * args.K + (size_t)kb * KB + ch * 8) * 2);
            *reinterpret_cast<uint4*>(bst + rr * 128 + ((ch ^ (rr & 7)) << 4)) = v;
          }
          ptx::fence_proxy_async_smem();
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(raw_empty(rs));   // after the values were used: the reads are complete for certain
          ptx::mbar_arrive(a_full(as));
        }
      }
    }
  } else if (warp >= C::FIRST_EPI) {
    // ------------------------------------------------------------ epilogue warps
    const int e = warp - C::FIRST_EPI;
    const int quarter = warp & 3;              // TMEM lanes 32*quarter .. +31 (a warp may only touch its own quarter)
    const int part = e >> 2;                   // which slice of the accumulator columns
    const int etid = e * 32 + lane;
    const int row = 8 * (4 * (lane >> 3) + quarter) + (lane & 7);
    constexpr int MY_COLS = C::MY_COLS;
    bool ok = true;
    int staged_chunk = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int mtok_shift = FEW ? 31 - __clz(mtok) : 0;   // mtok is a power of two
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int in_ = it / args.items_m, im = it - in_ * args.items_m;
      const int row0 = in_ * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      if (in_ != staged_chunk) {
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        stage_meta<uint16_t, SCALE_PITCH>(scaleT, args.scale, row0, nrows, args.gpr, etid, E * 32);
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        staged_chunk = in_;
      }
      float running[MY_COLS];
#pragma unroll
      for (int c = 0; c < MY_COLS; ++c) running[c] = 0.f;
      const bool live = row < nrows;
      const int n_safe = live ? row : 0;
      for (int ps = 0; ps < periods_per_item && ok; ps += SET) {
        const int set = acc / SET;
        if (!(ok = warp_wait(acc_full(set), acc_phase, 8))) break;
        ptx::tc_fence_after_sync();
        const int nvalid = min(SET, periods_per_item - ps);
#pragma unroll
        for (int a = 0; a < SET; ++a) {
          if (a < nvalid) {
            const int pi = ps + a;
            const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((acc + a) * N_MMA + part * MY_COLS);
            const int g0 = pi * args.G;
            float s;
            if (!FEW) s = bits_to_f32<F16>((uint32_t)scaleT[min(g0, args.gpr - 1) * SCALE_PITCH + n_safe]);
#pragma unroll
            for (int c0 = 0; c0 < MY_COLS / 16; ++c0) {
              uint32_t r[16];
              ptx::tmem_ld_32x32b_x16(t_addr + (uint32_t)(c0 * 16), r);
              ptx::tmem_ld_wait_16(r);
              if (a == nvalid - 1 && c0 == MY_COLS / 16 - 1) {   // the set's last columns are in registers: hand the set back
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(acc_empty(set));
              }
              if (FEW) {
                // column c = g_local * mtok + token; running[] stays indexed by column so that every index is a constant
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                  int g = g0 + (c >> mtok_shift);
                  if (g >= args.gpr) g = args.gpr - 1;   // columns of groups past K hold zeros
                  const float sg = bits_to_f32<F16>((uint32_t)scaleT[g * SCALE_PITCH + n_safe]);
                  running[c] = fmaf(sg, __uint_as_float(r[c]), running[c]);
                }
              } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) running[c0 * 16 + c] = fmaf(s, __uint_as_float(r[c]), running[c0 * 16 + c]);
              }
            }
          }
        }
        acc += SET;
        if (acc == NACC) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) break;
      // ---- store: y[m][row0 + row] = bf16(sum + bias)
      if (live) {
        const int n = row0 + row;
        const float b = args.bias ? args.bias[n] : 0.f;
        if (FEW) {
          // fold the G group slots of each token: column c holds token c & (mtok - 1)
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            if (m < mtok && m < args.M) {
              float v = 0.f;
#pragma unroll
              for (int c = 0; c < 16; ++c)
                if ((c & (mtok - 1)) == m) v += running[c];
              args.y[(size_t)m * args.N + n] = f32_to_bits<F16>(v + b);
            }
          }
        } else {
          const int m0 = im * MT + part * MY_COLS;
#pragma unroll
          for (int c = 0; c < MY_COLS; ++c) {
            const int m = m0 + c;
            if (m < args.M) args.y[(size_t)m * args.N + n] = f32_to_bits<F16>(running[c] + b);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, (uint32_t)TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && args.status != nullptr) atomicCAS(args.status, 0, *abort_flag);
}

template <int MT, bool F16>
int launch_umma(const CUtensorMap& tw, const CUtensorMap& tx, UmmaArgs a, int grid, cudaStream_t stream) {
  using C = Cfg<MT>;
  const int x_bytes = MT == 0 ? a.mtok * a.K * 2 : 0;
  // raw ring: as deep as shared memory allows (each stage carries 256 k of every row in flight), at most 8
  a.raw_stages = MAX_RAW;
  while (a.raw_stages > 2 && C::total(a.raw_stages, a.gpr, x_bytes) > 227 * 1024) --a.raw_stages;
  const int smem = C::total(a.raw_stages, a.gpr, x_bytes);
  if (smem > 227 * 1024) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 tensor-core kernel: shared memory does not hold two raw stages");
  a.idesc = ptx::make_idesc(1u, F16 ? 0u : 1u, F16 ? 0u : 1u, (uint32_t)TILE_ROWS, (uint32_t)C::N_MMA);  // f32 accumulate
  {
    // issuers in use: drain periods go round them, and a period's k-blocks occupy consecutive A stages; the ring of AS
    // stages must hold a whole number of rounds, and periods must not straddle items
    const int kbpp = a.G * a.kpg;
    int ni = C::NI;
    if (C::AS % kbpp != 0 || a.num_kb % kbpp != 0) ni = 1;
    else
      while (ni > 1 && (C::AS / kbpp) % ni != 0) ni /= 2;
    a.ni = ni;
  }
  auto kfn = a16_w4_umma_kernel<MT, F16>;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, tw, tx, a));
  return B200Q_OK;
}


// ---------------------------------------------------------------------------------------------------------------
// Few-token form (M <= 4): the kernel is bound by streaming and converting the weights, and a single MMA-issuing
// thread cannot keep up with one small MMA every ~28 cycles next to two dozen busy warps.  So there is no central
// issuer: the dequantisation warps form FW teams of four (one warp per TMEM lane quarter); team t owns the k-blocks
// j with j mod FW == t, two TMEM stages of A, two window buffers of B and ITS OWN 16 accumulator columns.  When the
// four quarters of a k-block have stored their rows, the team's quarter-0 warp issues its four MMAs and commits them.
// MMAs of different teams never touch the same accumulator columns, so their order does not matter; the epilogue adds
// the FW column sets of a period before it applies the group scales.
struct FewCfg {
  static constexpr int FW = 5;                       // teams
  static constexpr int E = 4;                        // epilogue warps, one per lane quarter
  static constexpr int NTHREADS = (4 + 4 * FW + E) * 32;   // 896
  static constexpr int AS = 2 * FW;                  // A stages in TMEM, B window buffers in shared memory
  static constexpr int ACC_COLS = FW * 16;           // accumulator columns per buffer
  static constexpr int A_COL0 = TMEM_COLS - AS * A_COLS;
  static constexpr int B_STAGE_BYTES = 32 * 128;
  static constexpr int FIRST_DQ = 4, FIRST_EPI = 4 + 4 * FW;
  static_assert(2 * ACC_COLS <= A_COL0, "accumulators and A stages share 512 columns");
  static constexpr int NUM_BARS = 2 * MAX_RAW + 2 * AS + 4 + 2;
  __host__ __device__ static int b_off(int rs) { return rs * RAW_STAGE_BYTES; }
  __host__ __device__ static int bar_off(int rs) { return b_off(rs) + AS * B_STAGE_BYTES; }
  __host__ __device__ static int misc_off(int rs) { return bar_off(rs) + NUM_BARS * 8; }
  __host__ __device__ static int meta_off(int rs) { return (misc_off(rs) + 16 + 127) & ~127; }
  __host__ __device__ static int x_off(int rs, int gpr) { return meta_off(rs) + ((gpr * (SCALE_PITCH * 2 + ZP_PITCH) + 15) & ~15); }
  __host__ __device__ static int total(int rs, int gpr, int x_bytes) { return x_off(rs, gpr) + x_bytes + 1024; }
};

__global__ void __launch_bounds__(FewCfg::NTHREADS, 1)
a16_w4_umma_few_kernel(const __grid_constant__ CUtensorMap tmap_w, const UmmaArgs args) {
  using C = FewCfg;
  constexpr int FW = C::FW, E = C::E, AS = C::AS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int RS = args.raw_stages;              // a power of two
  const int rs_shift = 31 - __clz(RS);
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int b_off = C::b_off(RS), misc_off = C::misc_off(RS), meta_off = C::meta_off(RS);
  const uint32_t bar_base = smem_base + (uint32_t)C::bar_off(RS);
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto raw_empty = [&](int s) { return bar_base + 8u * (MAX_RAW + s); };
  auto a_ready = [&](int s) { return bar_base + 8u * (2 * MAX_RAW + s); };
  auto a_free = [&](int s) { return bar_base + 8u * (2 * MAX_RAW + AS + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * MAX_RAW + 2 * AS + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * MAX_RAW + 2 * AS + 2 + a); };
  const uint32_t dq_sync_bar = bar_base + 8u * (2 * MAX_RAW + 2 * AS + 4), epi_sync_bar = dq_sync_bar + 8u;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);
  uint16_t* scaleT = reinterpret_cast<uint16_t*>(smem + meta_off);
  uint8_t* zpT = smem + meta_off + args.gpr * SCALE_PITCH * 2;
  uint8_t* xs = smem + C::x_off(RS, args.gpr);   // xs[m][K] bf16, 16-byte pieces in the nibble-pair order of A

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto role_sync = [&](uint32_t bar, uint32_t& count, int where) -> bool {
    __syncwarp();
    bool ok_ = true;
    if (lane == 0) {
      ptx::mbar_arrive(bar);
      ok_ = ptx::mbar_wait_bounded_fast(bar, count & 1u, abort_flag, where, WAIT_NS);
    }
    ++count;
    ok_ = __shfl_sync(0xffffffffu, ok_, 0);
    return ok_;
  };
  // every lane of the warp runs the same wait (the barrier test is one warp instruction either way)
  auto warp_wait = [&](uint32_t bar, uint32_t parity, int where) -> bool {
    return ptx::mbar_wait_bounded_fast(bar, parity, abort_flag, where, WAIT_NS);
  };

  ptx::griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      ptx::mbar_init(raw_full(s), 1);
      ptx::mbar_init(raw_empty(s), 4 * RAW_KB);   // one arrival per (k-block, lane quarter)
    }
    for (int s = 0; s < AS; ++s) {
      ptx::mbar_init(a_ready(s), 4);              // the four quarters of the team
      ptx::mbar_init(a_free(s), 1);               // the team's MMAs have read the stage
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(acc_full(a), FW);            // every team closes every period
      ptx::mbar_init(acc_empty(a), E);
    }
    ptx::mbar_init(dq_sync_bar, 4 * FW);
    ptx::mbar_init(epi_sync_bar, E);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), (uint32_t)TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::griddep_wait();
  {
    // the window buffers start as zeros; only their live rows are ever rewritten
    uint4* b = reinterpret_cast<uint4*>(smem + b_off);
    for (int i = threadIdx.x; i < AS * C::B_STAGE_BYTES / 16; i += C::NTHREADS) b[i] = make_uint4(0u, 0u, 0u, 0u);
    // activations: rows past M are zeros
    const int pieces = args.mtok * (args.K >> 3);
    for (int i = threadIdx.x; i < pieces; i += C::NTHREADS) {
      const int m = i / (args.K >> 3), c = i - m * (args.K >> 3);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < args.M) v = __ldg(reinterpret_cast<const uint4*>(args.x + ((size_t)m * args.K + (size_t)c * 8) * 2));
      uint4 o;   // k order 0,4,1,5,2,6,3,7
      o.x = __byte_perm(v.x, v.z, 0x5410);
      o.y = __byte_perm(v.x, v.z, 0x7632);
      o.z = __byte_perm(v.y, v.w, 0x5410);
      o.w = __byte_perm(v.y, v.w, 0x7632);
      reinterpret_cast<uint4*>(xs)[i] = o;
    }
    ptx::fence_proxy_async_smem();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int items = args.items_n;
  const int item_begin = (int)((long long)blockIdx.x * items / gridDim.x);
  const int item_end = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);
  const int num_kb = args.num_kb;
  const int raws_per_item = (num_kb + RAW_KB - 1) / RAW_KB;
  const int kb_per_period = args.G * args.kpg;
  const int periods_per_item = (num_kb + kb_per_period - 1) / kb_per_period;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: packed weights
    if (lane == 0) {
      bool ok = true;
      int rs = 0;
      uint32_t rphase = 0;
      for (int it = item_begin; it < item_end && ok; ++it) {
        const int row0 = it * args.rows_item;
        const int nrows = min(args.rows_item, args.N - row0);
        const int boxes = (nrows + 15) >> 4;
        for (int rsi = 0; rsi < raws_per_item; ++rsi) {
          ok = ptx::mbar_wait_bounded_fast(raw_empty(rs), rphase ^ 1u, abort_flag, 1, WAIT_NS);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(raw_full(rs), (uint32_t)boxes * 16u * 128u);
          const uint32_t dst = smem_base + (uint32_t)rs * RAW_STAGE_BYTES;
          for (int b = 0; b < boxes; ++b) ptx::tma_load_2d(dst + (uint32_t)b * 2048u, &tmap_w, raw_full(rs), rsi * 128, row0 + b * 16);
          const int nreal = min(RAW_KB, num_kb - rsi * RAW_KB);
          if (nreal < RAW_KB) ptx::mbar_arrive_n(raw_empty(rs), (uint32_t)(4 * (RAW_KB - nreal)));
          if (++rs == RS) {
            rs = 0;
            rphase ^= 1u;
          }
        }
      }
    }
  } else if (warp >= C::FIRST_DQ && warp < C::FIRST_EPI) {
    // ------------------------------------------------------------ dequantisation teams (quarter 0 also issues the MMAs)
    const int dq = warp - C::FIRST_DQ;
    const int quarter = warp & 3;
    const int team = dq >> 2;
    const int dtid = dq * 32 + lane;
    const int row = 8 * (4 * (lane >> 3) + quarter) + (lane & 7);   // row of the work item held by this TMEM lane
    bool ok = true;
    int staged_item = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int live_row0 = (args.G - 1) * mtok;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)C::A_COL0;
    const uint64_t bdesc0 = ptx::make_smem_desc_kmajor(smem_base + (uint32_t)b_off, 1024, 2);
    const uint32_t b_hi = (uint32_t)(bdesc0 >> 32), b_lo0 = (uint32_t)bdesc0;
    const uint32_t idesc = args.idesc;
    const int kpg = args.kpg;
    const int pshift = (kb_per_period & (kb_per_period - 1)) == 0 ? 31 - __clz(kb_per_period) : -1;
    uint32_t cnt = 0;   // k-blocks this team has handled: stage 2 * team + (cnt & 1), phase (cnt >> 1) & 1
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int row0 = it * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      if (it != staged_item) {
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;  // everyone is done with the previous item's
        stage_meta<uint8_t, ZP_PITCH>(zpT, args.zp, row0, nrows, args.gpr, dtid, 4 * FW * 32);
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;
        staged_item = it;
      }
      const bool live = row < nrows;
      const int jbase = (it - item_begin) * num_kb, rbase = (it - item_begin) * raws_per_item;
      const int pbase = (it - item_begin) * periods_per_item;
      int kb = team - jbase % FW;
      if (kb < 0) kb += FW;
      int pcur = -1;   // issuer: the last period this team has entered
      // issuer: a period in which the team has no k-block still needs its arrival (after the buffer's previous use)
      auto close_empty_periods = [&](int from, int to) -> bool {
        for (int p = from; p < to; ++p) {
          const int pd = pbase + p, buf = pd & 1;
          if (!warp_wait(acc_empty(buf), (((uint32_t)(pd >> 1)) & 1u) ^ 1u, 3)) return false;
          if (lane == 0) ptx::mbar_arrive(acc_full(buf));
        }
        return true;
      };
      for (; kb < num_kb && ok; kb += FW, ++cnt) {
        const int stage = 2 * team + (int)(cnt & 1u);
        const uint32_t sphase = (cnt >> 1) & 1u;
        const int r = rbase + (kb >> 2), rs = r & (RS - 1), sub = kb & (RAW_KB - 1);
        if (!(ok = warp_wait(raw_full(rs), (uint32_t)(r >> rs_shift) & 1u, 6))) break;
        uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = w0;
        if (live) {
          const uint8_t* rrow = smem + (size_t)rs * RAW_STAGE_BYTES + row * 128;
          w0 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub) ^ (row & 7)) << 4));
          w1 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub + 1) ^ (row & 7)) << 4));
        }
        const int g = kpg == 1 ? kb : kb / kpg;
        const uint32_t z = live ? zpT[g * ZP_PITCH + row] : 0u;
        const uint32_t negz = __byte_perm(z, 0xC3u, 0x4040);  // bf16x2 {-(128 + zp), -(128 + zp)}: 0xC300 | zp
        if (!(ok = warp_wait(a_free(stage), sphase ^ 1u, 7))) break;
        ptx::tc_fence_after_sync();
        const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t o[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t p[4];
            dequant_word(ww[4 * h + q], negz, p);   // k order 0,4,1,5,2,6,3,7 inside every 8, like B
            o[4 * q + 0] = p[0];
            o[4 * q + 1] = p[1];
            o[4 * q + 2] = p[2];
            o[4 * q + 3] = p[3];
          }
          ptx::tmem_st_32x32b_x16(t_lane + (uint32_t)(stage * A_COLS + 16 * h), o);
        }
        if (quarter == 0) {
          // this k-block's activations from the resident copy into the live rows of the team's window buffer
          uint8_t* bst = smem + b_off + (size_t)stage * C::B_STAGE_BYTES;
          if (lane < mtok * 8) {
            const int m = lane >> 3, ch = lane & 7, rr = live_row0 + m;
            const uint4 v = *reinterpret_cast<const uint4*>(xs + ((size_t)m * args.K + (size_t)kb * KB + ch * 8) * 2);
            *reinterpret_cast<uint4*>(bst + rr * 128 + ((ch ^ (rr & 7)) << 4)) = v;
          }
          ptx::fence_proxy_async_smem();
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(raw_empty(rs));   // after the values were used: the reads are complete for certain
          ptx::mbar_arrive(a_ready(stage));
        }
        if (quarter == 0) {
          // ---- issue this k-block's MMAs into the team's accumulator columns
          const int pi = pshift >= 0 ? (kb >> pshift) : kb / kb_per_period, pd = pbase + pi, buf = pd & 1;
          bool first = false;
          if (pi != pcur) {
            if (!(ok = close_empty_periods(pcur + 1, pi))) break;
            if (!(ok = warp_wait(acc_empty(buf), (((uint32_t)(pd >> 1)) & 1u) ^ 1u, 3))) break;
            first = true;
            pcur = pi;
          }
          if (!(ok = warp_wait(a_ready(stage), sphase, 4))) break;
          ptx::tc_fence_after_sync();
          if (lane == 0) {
            const int g_local = g - pi * args.G;
            const uint32_t b_lo = b_lo0 + (uint32_t)stage * (C::B_STAGE_BYTES >> 4) + (uint32_t)((args.G - 1 - g_local) * mtok) * 8u;
            ptx::umma_kblock_f16_ts(tmem_base + (uint32_t)(buf * C::ACC_COLS + team * 16), tmem_base + (uint32_t)(C::A_COL0 + stage * A_COLS),
                                    b_lo, b_hi, idesc, first ? 0u : 1u);
            ptx::umma_commit(a_free(stage));
            // the team's last k-block of this period: its part of the accumulator is complete when these MMAs are
            if (kb + FW >= num_kb || kb + FW >= (pi + 1) * kb_per_period) ptx::umma_commit(acc_full(buf));
          }
          __syncwarp();
        }
      }
      if (ok && quarter == 0) ok = close_empty_periods(pcur + 1, periods_per_item);
    }
  } else if (warp >= C::FIRST_EPI) {
    // ------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;
    const int etid = (warp - C::FIRST_EPI) * 32 + lane;
    const int row = 8 * (4 * (lane >> 3) + quarter) + (lane & 7);
    bool ok = true;
    int staged_item = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int mtok_shift = 31 - __clz(mtok);   // mtok is a power of two
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int row0 = it * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      if (it != staged_item) {
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        stage_meta<uint16_t, SCALE_PITCH>(scaleT, args.scale, row0, nrows, args.gpr, etid, E * 32);
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        staged_item = it;
      }
      float running[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) running[c] = 0.f;
      const bool live = row < nrows;
      const int n_safe = live ? row : 0;
      const int pbase = (it - item_begin) * periods_per_item;
      for (int pi = 0; pi < periods_per_item && ok; ++pi) {
        const int pd = pbase + pi, buf = pd & 1;
        if (!(ok = warp_wait(acc_full(buf), ((uint32_t)(pd >> 1)) & 1u, 8))) break;
        ptx::tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * C::ACC_COLS);
        float sum[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) sum[c] = 0.f;
        // the column sets of the teams that had a k-block in this period (a set without one holds old values)
        const int lo = pi * kb_per_period, hi = min(lo + kb_per_period, num_kb);
        const int jlo = ((it - item_begin) * num_kb + lo) % FW;   // team of the period's first k-block
#pragma unroll
        for (int t = 0; t < FW; ++t) {
          int d = t - jlo;
          if (d < 0) d += FW;
          if (lo + d < hi) {   // same for every thread
            uint32_t r[16];
            ptx::tmem_ld_32x32b_x16(t_addr + (uint32_t)(t * 16), r);
            ptx::tmem_ld_wait_16(r);
#pragma unroll
            for (int c = 0; c < 16; ++c) sum[c] += __uint_as_float(r[c]);
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty(buf));
        // column c = g_local * mtok + token; running[] stays indexed by column so that every index is a constant
        const int g0 = pi * args.G;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          int g = g0 + (c >> mtok_shift);
          if (g >= args.gpr) g = args.gpr - 1;   // columns of groups past K hold zeros
          const float s = __uint_as_float((uint32_t)scaleT[g * SCALE_PITCH + n_safe] << 16);
          running[c] = fmaf(s, sum[c], running[c]);
        }
      }
      if (!ok) break;
      if (live) {
        const int n = row0 + row;
        const float b = args.bias ? args.bias[n] : 0.f;
        // fold the G group slots of each token: column c holds token c & (mtok - 1)
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < mtok && m < args.M) {
            float v = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if ((c & (mtok - 1)) == m) v += running[c];
            args.y[(size_t)m * args.N + n] = f32_to_bf16_bits_ref(v + b);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, (uint32_t)TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && args.status != nullptr) atomicCAS(args.status, 0, *abort_flag);
}

int launch_umma_few(const CUtensorMap& tw, UmmaArgs a, int grid, cudaStream_t stream) {
  using C = FewCfg;
  const int x_bytes = a.mtok * a.K * 2;
  a.raw_stages = MAX_RAW;   // a power of two: 8, 4 or 2
  while (a.raw_stages > 2 && C::total(a.raw_stages, a.gpr, x_bytes) > 227 * 1024) a.raw_stages >>= 1;
  const int smem = C::total(a.raw_stages, a.gpr, x_bytes);
  if (smem > 227 * 1024) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 tensor-core kernel: shared memory does not hold two raw stages");
  a.idesc = ptx::make_idesc(1u, 1u, 1u, (uint32_t)TILE_ROWS, 16u);
  auto kfn = a16_w4_umma_few_kernel;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::NTHREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, tw, a));
  return B200Q_OK;
}

}  // namespace

int a16_w4_umma_supported(long long M, int N, int K, int group, const char** why) {
  const char* w = nullptr;
  if (M < 1 || M > 0x7fffffffLL) w = "M out of range";
  else if (N < 1) w = "empty N";
  else if (K % KB != 0) w = "K must be a multiple of 64";
  else if (group < KB || group % KB != 0 || K % group != 0) w = "the group size must be a multiple of 64 that divides K";
  else if ((K / 2) % 16 != 0) w = "the weight row pitch must be a multiple of 16 bytes";
  else if (Cfg<32>::total(2, K / group, 0) > 227 * 1024) w = "the scales and zero points of one 128-row tile do not fit in shared memory";
  if (why) *why = w;
  return w == nullptr;
}

int a16_w4_umma_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       long long M, int N, int K, int group, int* status, cudaStream_t stream, bool f16) {
  const char* why = nullptr;
  if (!a16_w4_umma_supported(M, N, K, group, &why)) return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 tensor-core kernel: %s", why);
  if ((reinterpret_cast<uintptr_t>(wq) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return set_error(B200Q_ERR_INVALID, "a16 w4: weights and activations must be 16-byte aligned");
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  UmmaArgs a{};
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
  a.num_kb = K / KB;
  a.kpg = group / KB;
  a.status = status;
  {
    static const int dbg = [] {
      const char* v = getenv("B200Q_UMMA_DEBUG");
      return v ? atoi(v) : 0;
    }();
    a.debug = dbg;
  }
  // few-token form: up to 4 tokens whose activations fit in shared memory next to two raw stages
  const int mtok_few = M <= 1 ? 1 : M <= 2 ? 2 : 4;
  const bool few = !f16 && M <= 4 && FewCfg::total(2, a.gpr, mtok_few * K * 2) <= 227 * 1024;   // (the few-token form is built for bf16)
  int mt = 0;
  if (few) {
    a.mtok = mtok_few;
    a.G = 16 / a.mtok;
    a.items_m = 1;
  } else {
    mt = M <= 32 ? 32 : M <= 64 ? 64 : 128;
    // many groups per row leave less shared memory for the activation ring: narrower token tiles then
    if (mt == 128 && Cfg<128>::total(2, a.gpr, 0) > 227 * 1024) mt = 64;
    if (mt == 64 && Cfg<64>::total(2, a.gpr, 0) > 227 * 1024) mt = 32;
    a.mtok = mt;
    a.G = 1;
    a.items_m = (int)((M + mt - 1) / mt);
  }
  // rows per work item: full 128-row tiles when they fill the SMs twice over, else row chunks (multiples of 16) sized
  // so that every SM gets one
  const long long full_tiles = (long long)((N + TILE_ROWS - 1) / TILE_ROWS) * a.items_m;
  if (full_tiles >= 2LL * sms) {
    a.rows_item = TILE_ROWS;
  } else {
    long long per = ((long long)N * a.items_m + sms - 1) / sms;   // rows x token tiles spread over the SMs
    per = (per + 15) / 16 * 16;
    if (per > TILE_ROWS) per = TILE_ROWS;
    if (per < 16) per = 16;
    a.rows_item = (int)per;
  }
  a.items_n = (N + a.rows_item - 1) / a.rows_item;
  const long long items = (long long)a.items_n * a.items_m;
  const int grid = (int)(items < sms ? items : sms);

  CUtensorMap tw, tx;
  {
    const uint64_t dims[2] = {(uint64_t)(K / 2), (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)(K / 2)};
    // 16-row boxes (one box of rows_item rows per raw stage was measured: no faster below 64 tokens, slower above)
    a.raw_box_rows = 16;
    const uint32_t box[2] = {128u, (uint32_t)a.raw_box_rows};
    B200Q_TRY(make_tmap_u8(&tw, wq, 2, dims, strides, box));
  }
  if (few) return launch_umma_few(tw, a, grid, stream);
  {
    const uint64_t dims[2] = {(uint64_t)K * 2, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {128u, (uint32_t)mt};
    B200Q_TRY(make_tmap_u8(&tx, x, 2, dims, strides, box));
  }
  if (f16) {
    if (mt == 32) return launch_umma<32, true>(tw, tx, a, grid, stream);
    if (mt == 64) return launch_umma<64, true>(tw, tx, a, grid, stream);
    return launch_umma<128, true>(tw, tx, a, grid, stream);
  }
  if (mt == 32) return launch_umma<32, false>(tw, tx, a, grid, stream);
  if (mt == 64) return launch_umma<64, false>(tw, tx, a, grid, stream);
  return launch_umma<128, false>(tw, tx, a, grid, stream);
}

}  // namespace b200q
