// A16MatMul with 4-bit group-quantized weights on the 5th-generation tensor cores: the packed weights are dequantised
// in registers, written to shared memory as the bf16 A operand of tcgen05.mma (kind::f16, fp32 accumulation in TMEM),
// and never exist in global memory in any wider form.
//
// Semantics: tpu::A16MatMulOp::inference, static w4 path with w_transpose
// (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246): weight bytes [N, K/2], even k in the low
// nibble, W[n,k] = (q - zp[n, k/g]) * scale[n, k/g], y = bf16(x * W^T (+ bias)) with fp32 accumulation.  The
// reference keeps W in fp32 (A16MatMul.cpp:190-198 does not round it); so does this kernel in effect: the tensor
// cores multiply the exact small integers (q - zp) with the bf16 activations, and the group scale multiplies the
// fp32 partial sum of each group afterwards.
//
// The product is computed transposed, D[n, m] = sum_k A[n, k] * B[m, k]: the 128 TMEM lanes are output channels,
// the columns are tokens.  One persistent CTA per SM, 20 warps:
//   warp 0       TMA producer: packed weights, boxes of 16 rows x 128 bytes (= 256 k) with the 128-byte swizzle into
//                a ring of raw stages; in the many-token form also the activation tile of each k-block.
//   warp 1       owns TMEM, issues the MMAs (one thread): per k-block of 64 k four MMAs 128 x N x 16.
//   warps 4-11   dequantisation, four teams of two warps; team t converts k-block t of every raw stage, so four
//                k-blocks are in the making at any time: one 32-bit word (8 nibbles) -> 128 + q as bf16 by the bit
//                trick, minus (128 + zp) in one packed bf16 FMA, 16 bytes of A, written as rows of the 128-byte
//                swizzled K-major layout.  In the few-token form the team also writes the k-block's activations
//                into the B operand.
//   warps 12-19  epilogue: drain the accumulator of each period, running[n][m] += scale[n][g] * partial; at the end of
//                a work item add the bias, round to bf16 and store y[m][n].
//
// Groups and columns.  The group scale cannot ride through the MMA, so partial sums of different groups must stay
// apart.  With many tokens (M > 16) the accumulator is drained after every group (two TMEM buffers alternate).  With
// few tokens the accumulator has spare columns: column j = g_local * MTOK + m belongs to group g_local of the current
// period of G = 16 / MTOK groups, and the B operand of a k-block of group g_local is zero except in its MTOK rows.  That
// operand is a window into one small buffer, (G-1)*MTOK zero rows | the MTOK activation rows | (G-1)*MTOK zero rows,
// starting (G-1-g_local)*MTOK rows into it, so only the MTOK live rows are rewritten per k-block.  One drain then serves G
// groups (for one token and K = 4096: four drains per row instead of 64).
//
// Every mbarrier wait is bounded (2 s); a wait that runs out leaves its site code in a shared flag, every role
// unwinds, TMEM is freed and *status receives the code.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "a16.h"
#include "igemm.h"
#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200q {
namespace {

constexpr int TILE_ROWS = 128;           // output channels per work item = MMA M
constexpr int KB = 64;                   // k per k-block: 64 bf16 = one 128-byte swizzle span
constexpr int RAW_KB = 4;                // k-blocks per raw stage (128 bytes of nibbles per row)
constexpr int RAW_STAGE_BYTES = TILE_ROWS * 128;
constexpr int A_STAGE_BYTES = TILE_ROWS * 128;
constexpr int MAX_STAGES = 8;
constexpr int DQ_WARPS = 8, EPI_WARPS = 8, TEAM_THREADS = 64;  // four teams of two warps
constexpr int FIRST_DQ_WARP = 4, FIRST_EPI_WARP = 12;
constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;  // 640
constexpr int SCALE_PITCH = TILE_ROWS + 2;   // scaleT[g][n], bf16: transposed so that lanes (rows) read one group conflict-free
constexpr int ZP_PITCH = TILE_ROWS + 4;      // zpT[g][n], bytes
constexpr uint64_t WAIT_NS = 2000000000ull;

struct UmmaArgs {
  const uint8_t* x;       // bf16 [M][K]
  const uint16_t* scale;  // bf16 [N][gpr]
  const uint8_t* zp;      // u8 [N][gpr]
  const float* bias;      // [N] or null
  uint16_t* y;            // bf16 [M][N]
  int M, N, K, group, gpr;
  int num_kb;             // K / 64
  int kpg;                // k-blocks per group
  int mtok;               // few-token form: token rows per group slot (1, 2, 4, 8 or 16); many-token form: tile width
  int G;                  // groups per drain period
  int n_mma;              // MMA N = accumulator columns
  int rows_item;          // output channels per work item (multiple of 16, <= 128)
  int items_n, items_m;   // work items: items_n row chunks x items_m token tiles
  int raw_stages, op_stages;  // ring depths (chosen by the host so that everything fits in shared memory)
  uint32_t idesc;
  int* status;
};

// Shared-memory plan, the same on host and device: raw ring | A ring | B ring | barriers | misc | scaleT | zpT
template <int MT_LARGE>
struct Smem {
  // MT_LARGE == 0: few-token form (B written by the dequantisation teams, 32-row window buffer); else B by TMA
  static constexpr int B_STAGE_BYTES = MT_LARGE == 0 ? 32 * 128 : MT_LARGE * 128;
  static constexpr int NUM_BARS = 4 * MAX_STAGES + 6;
  __host__ __device__ static int a_off(int raw_stages) { return raw_stages * RAW_STAGE_BYTES; }
  __host__ __device__ static int b_off(int raw_stages, int op_stages) { return a_off(raw_stages) + op_stages * A_STAGE_BYTES; }
  __host__ __device__ static int bar_off(int raw_stages, int op_stages) { return b_off(raw_stages, op_stages) + op_stages * B_STAGE_BYTES; }
  __host__ __device__ static int misc_off(int raw_stages, int op_stages) { return bar_off(raw_stages, op_stages) + NUM_BARS * 8; }
  __host__ __device__ static int meta_off(int raw_stages, int op_stages) { return (misc_off(raw_stages, op_stages) + 16 + 127) & ~127; }
  __host__ __device__ static int total(int raw_stages, int op_stages, int gpr) {
    return meta_off(raw_stages, op_stages) + gpr * (SCALE_PITCH * 2 + ZP_PITCH) + 1024;
  }
};

// 8 nibbles of `w` (k0..k7, k0 lowest) -> four bf16x2 words {q_j - zp, q_(j+4) - zp}, j = 0..3
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t negz, uint32_t (&p)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // {128 + q_j, 128 + q_(j+4)}
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(p[j]) : "r"(t), "r"(0x3F803F80u), "r"(negz));  // exact: small integers
  }
}

template <int MT_LARGE>
__global__ void __launch_bounds__(THREADS, 1)
a16_w4_umma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const UmmaArgs args) {
  using L = Smem<MT_LARGE>;
  constexpr bool FEW = MT_LARGE == 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int RS = args.raw_stages, OS = args.op_stages;
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int a_off = L::a_off(RS), b_off = L::b_off(RS, OS), misc_off = L::misc_off(RS, OS);
  const uint32_t bar_base = smem_base + (uint32_t)L::bar_off(RS, OS);
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto raw_empty = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto op_full = [&](int s) { return bar_base + 8u * (2 * MAX_STAGES + s); };
  auto op_empty = [&](int s) { return bar_base + 8u * (3 * MAX_STAGES + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (4 * MAX_STAGES + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (4 * MAX_STAGES + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);
  uint16_t* scaleT = reinterpret_cast<uint16_t*>(smem + L::meta_off(RS, OS));
  uint8_t* zpT = smem + L::meta_off(RS, OS) + args.gpr * SCALE_PITCH * 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t dq_sync_bar = bar_base + 8u * (4 * MAX_STAGES + 4), epi_sync_bar = bar_base + 8u * (4 * MAX_STAGES + 5);
  // Meeting point of the 8 warps of a role on an mbarrier (one arrival per warp), with the same bounded wait as
  // every other wait of the kernel: a plain bar.sync would hang if one warp had already given up.
  auto role_sync = [&](uint32_t bar, uint32_t& count, int where) -> bool {
    __syncwarp();
    bool ok_ = true;
    if (lane == 0) {
      ptx::mbar_arrive(bar);
      ok_ = ptx::mbar_wait_bounded(bar, count & 1u, abort_flag, where, WAIT_NS);
    }
    ++count;
    ok_ = __shfl_sync(0xffffffffu, ok_, 0);
    return ok_;
  };
  const int tmem_cols = 2 * args.n_mma < 32 ? 32 : 2 * args.n_mma;  // power of two: n_mma is 16, 32, 64 or 128

  ptx::griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      ptx::mbar_init(raw_full(s), 1);
      ptx::mbar_init(raw_empty(s), DQ_WARPS);
    }
    for (int s = 0; s < OS; ++s) {
      ptx::mbar_init(op_full(s), FEW ? 2 : 3);  // the two warps of a team (+ the TMA producer's activation tile)
      ptx::mbar_init(op_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(acc_full(a), 1);
      ptx::mbar_init(acc_empty(a), EPI_WARPS);
    }
    ptx::mbar_init(dq_sync_bar, DQ_WARPS);
    ptx::mbar_init(epi_sync_bar, EPI_WARPS);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_w);
    if (!FEW) ptx::prefetch_tensormap(&tmap_x);
  }
  if (FEW) {
    // the window buffers start as zeros; only their live rows are ever rewritten
    uint4* b = reinterpret_cast<uint4*>(smem + b_off);
    for (int i = threadIdx.x; i < OS * L::B_STAGE_BYTES / 16; i += THREADS) b[i] = make_uint4(0u, 0u, 0u, 0u);
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), (uint32_t)tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // work items of this CTA: a contiguous range, token tiles innermost (consecutive items share their weight rows'
  // scales and zero points).  Ring positions derive from running counts: k-block j of the CTA uses operand stage
  // j % OS in phase (j / OS) & 1, raw stage r likewise.
  const int items = args.items_n * args.items_m;
  const int item_begin = (int)((long long)blockIdx.x * items / gridDim.x);
  const int item_end = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);
  const int num_kb = args.num_kb;
  const int raws_per_item = (num_kb + RAW_KB - 1) / RAW_KB;
  const int kb_per_period = args.G * args.kpg;
  const int periods_per_item = (num_kb + kb_per_period - 1) / kb_per_period;
  ptx::griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = item_begin; it < item_end && ok; ++it) {
        const int in_ = it / args.items_m, im = it - in_ * args.items_m;
        const int row0 = in_ * args.rows_item;
        const int nrows = min(args.rows_item, args.N - row0);
        const int boxes = (nrows + 15) >> 4;
        const int jbase = (it - item_begin) * num_kb, rbase = (it - item_begin) * raws_per_item;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if ((kb & (RAW_KB - 1)) == 0) {
            const int r = rbase + kb / RAW_KB, rs = r % RS;
            ok = ptx::mbar_wait_bounded(raw_empty(rs), (((uint32_t)(r / RS)) & 1u) ^ 1u, abort_flag, 1, WAIT_NS);
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(raw_full(rs), (uint32_t)boxes * 16u * 128u);
            const uint32_t dst = smem_base + (uint32_t)rs * RAW_STAGE_BYTES;
            for (int b = 0; b < boxes; ++b)
              ptx::tma_load_2d(dst + (uint32_t)b * 2048u, &tmap_w, raw_full(rs), (kb / RAW_KB) * 128, row0 + b * 16);
          }
          if (!FEW) {
            const int j = jbase + kb, os = j % OS;
            ok = ptx::mbar_wait_bounded(op_empty(os), (((uint32_t)(j / OS)) & 1u) ^ 1u, abort_flag, 2, WAIT_NS);
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(op_full(os), (uint32_t)MT_LARGE * 128u);
            ptx::tma_load_2d(smem_base + (uint32_t)b_off + (uint32_t)os * L::B_STAGE_BYTES, &tmap_x, op_full(os), kb * 128,
                             im * MT_LARGE);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      const uint64_t desc0 = ptx::make_smem_desc_kmajor(smem_base + (uint32_t)a_off, 1024, 2);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)desc0;
      const uint32_t b_lo0 = (uint32_t)ptx::make_smem_desc_kmajor(smem_base + (uint32_t)b_off, 1024, 2);
      for (int it = item_begin; it < item_end && ok; ++it) {
        const int jbase = (it - item_begin) * num_kb, pbase = (it - item_begin) * periods_per_item;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          const int in_period = kb % kb_per_period;
          const int pd = pbase + kb / kb_per_period, acc = pd & 1;
          if (in_period == 0) {
            ok = ptx::mbar_wait_bounded(acc_empty(acc), (((uint32_t)(pd >> 1)) & 1u) ^ 1u, abort_flag, 3, WAIT_NS);
            if (!ok) break;
            ptx::tc_fence_after_sync();
          }
          const int j = jbase + kb, os = j % OS;
          ok = ptx::mbar_wait_bounded(op_full(os), ((uint32_t)(j / OS)) & 1u, abort_flag, 4, WAIT_NS);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * args.n_mma);
          const int g_local = in_period / args.kpg;
          // few-token form: the window starts (G - 1 - g_local) * mtok rows into the buffer
          const uint32_t b_row = FEW ? (uint32_t)((args.G - 1 - g_local) * args.mtok) : 0u;
          const uint32_t a_lo = a_lo0 + (uint32_t)os * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)os * (L::B_STAGE_BYTES >> 4) + b_row * (128u >> 4);
          ptx::umma_kblock_f16(d_tmem, a_lo, b_lo, desc_hi, desc_hi, args.idesc, in_period != 0 ? 1u : 0u);
          ptx::umma_commit(op_empty(os));
          if (in_period == kb_per_period - 1 || kb == num_kb - 1) ptx::umma_commit(acc_full(acc));
        }
      }
    }
  } else if (warp >= FIRST_DQ_WARP && warp < FIRST_EPI_WARP) {
    // ------------------------------------------------------------ dequantisation teams
    const int dq = warp - FIRST_DQ_WARP;          // 0..7
    const int dtid = dq * 32 + lane;              // 0..255
    const int team = dq >> 1;                     // converts k-block `team` of every raw stage
    const int ttid = (dq & 1) * 32 + lane;        // 0..63 inside the team
    bool ok = true;
    int staged_chunk = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int live_row0 = (args.G - 1) * mtok;    // few-token form: first live row of the window buffer
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int in_ = it / args.items_m;
      const int row0 = in_ * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      const int rows8 = (nrows + 7) & ~7;         // tasks are laid out over whole 8-row groups
      if (in_ != staged_chunk) {
        // zero points of this row chunk, transposed: zpT[g][n]
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;  // everyone is done with the previous chunk's
        const int total = nrows * args.gpr;
        for (int i = dtid; i < total; i += DQ_WARPS * 32) {
          const int n = i / args.gpr, g = i - n * args.gpr;
          zpT[g * ZP_PITCH + n] = __ldg(args.zp + (size_t)(row0 + n) * args.gpr + g);
        }
        if (!(ok = role_sync(dq_sync_bar, sync_count, 9))) break;
        staged_chunk = in_;
      }
      const int jbase = (it - item_begin) * num_kb, rbase = (it - item_begin) * raws_per_item;
      for (int rsi = 0; rsi < raws_per_item && ok; ++rsi) {
        const int r = rbase + rsi, rs = r % RS;
        const int kb = rsi * RAW_KB + team;
        const bool have = kb < num_kb;
        // few-token form: this k-block's activations (global memory; requested before the waits)
        uint4 xv[2];
        if (FEW && have) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c = ttid + TEAM_THREADS * u;   // 16-byte chunk: token c / 8, chunk c % 8
            xv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (c < mtok * 8 && (c >> 3) < args.M)
              xv[u] = __ldg(reinterpret_cast<const uint4*>(args.x + ((size_t)(c >> 3) * args.K + (size_t)kb * KB + (c & 7) * 8) * 2));
          }
        }
        if (lane == 0) ok = ptx::mbar_wait_bounded(raw_full(rs), ((uint32_t)(r / RS)) & 1u, abort_flag, 6, WAIT_NS);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        // a task = (row, half of the k-block): 16 bytes of nibbles -> 64 bytes of A.  Lanes of a quarter warp take
        // consecutive rows of one half, which keeps the swizzled reads and writes free of bank conflicts.
        constexpr int MAX_TASKS = 2 * TILE_ROWS / TEAM_THREADS;  // 4
        uint4 wv[MAX_TASKS];
        const uint8_t* rst = smem + (size_t)rs * RAW_STAGE_BYTES;
#pragma unroll
        for (int t = 0; t < MAX_TASKS; ++t) {
          const int task = ttid + TEAM_THREADS * t;
          const int half = task >= rows8 ? 1 : 0, row = task - half * rows8;
          wv[t] = make_uint4(0u, 0u, 0u, 0u);
          if (have && task < 2 * rows8)
            wv[t] = *reinterpret_cast<const uint4*>(rst + row * 128 + (((2 * team + half) ^ (row & 7)) << 4));
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(raw_empty(rs));   // this warp has read its part of the raw stage
        if (!have) continue;
        const int j = jbase + kb, os = j % OS;
        const int g = kb / args.kpg;
        if (lane == 0) ok = ptx::mbar_wait_bounded(op_empty(os), (((uint32_t)(j / OS)) & 1u) ^ 1u, abort_flag, 7, WAIT_NS);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        uint8_t* ast = smem + a_off + (size_t)os * A_STAGE_BYTES;
#pragma unroll
        for (int t = 0; t < MAX_TASKS; ++t) {
          const int task = ttid + TEAM_THREADS * t;
          if (task < 2 * rows8) {
            const int half = task >= rows8 ? 1 : 0, row = task - half * rows8;
            const uint32_t z = zpT[g * ZP_PITCH + row];
            const uint32_t negz = __byte_perm(z, 0xC3u, 0x4040);  // bf16x2 {-(128 + zp), -(128 + zp)}: 0xC300 | zp
            const uint32_t ww[4] = {wv[t].x, wv[t].y, wv[t].z, wv[t].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t p[4];
              dequant_word(ww[q], negz, p);
              uint4 o;
              if (FEW) {
                o = make_uint4(p[0], p[1], p[2], p[3]);   // k order 0,4,1,5,2,6,3,7 (B is written in the same order)
              } else {
                o.x = __byte_perm(p[0], p[1], 0x5410);    // natural k order: B arrives by TMA
                o.y = __byte_perm(p[2], p[3], 0x5410);
                o.z = __byte_perm(p[0], p[1], 0x7632);
                o.w = __byte_perm(p[2], p[3], 0x7632);
              }
              const int ch = half * 4 + q;   // logical 16-byte chunk of the A row
              *reinterpret_cast<uint4*>(ast + row * 128 + ((ch ^ (row & 7)) << 4)) = o;
            }
          }
        }
        if (FEW) {
          uint8_t* bst = smem + b_off + (size_t)os * L::B_STAGE_BYTES;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c = ttid + TEAM_THREADS * u;
            if (c < mtok * 8) {
              const int rr = live_row0 + (c >> 3), ch = c & 7;
              // the k order inside a 16-byte chunk follows the nibble-pair order of the A operand: 0,4,1,5,2,6,3,7
              uint4 o;
              o.x = __byte_perm(xv[u].x, xv[u].z, 0x5410);
              o.y = __byte_perm(xv[u].x, xv[u].z, 0x7632);
              o.z = __byte_perm(xv[u].y, xv[u].w, 0x5410);
              o.w = __byte_perm(xv[u].y, xv[u].w, 0x7632);
              *reinterpret_cast<uint4*>(bst + rr * 128 + ((ch ^ (rr & 7)) << 4)) = o;
            }
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(op_full(os));
      }
    }
  } else if (warp >= FIRST_EPI_WARP) {
    // ------------------------------------------------------------ epilogue warps
    const int e = warp - FIRST_EPI_WARP;       // 0..7
    const int quarter = warp & 3;              // TMEM lanes 32*quarter .. +31 (a warp may only touch its own quarter)
    const int chalf = e >> 2;                  // which half of the accumulator columns
    const int etid = e * 32 + lane;
    const int n_loc = quarter * 32 + lane;     // output channel inside the work item
    constexpr int MY_COLS = FEW ? 16 : MT_LARGE / 2;
    const bool active_warp = FEW ? (chalf == 0) : true;   // few-token form: one warp per quarter takes all 16 columns
    bool ok = true;
    int staged_chunk = -1;
    uint32_t sync_count = 0;
    const int mtok = args.mtok;
    const int mtok_shift = 31 - __clz(mtok);   // mtok is a power of two
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int in_ = it / args.items_m, im = it - in_ * args.items_m;
      const int row0 = in_ * args.rows_item;
      const int nrows = min(args.rows_item, args.N - row0);
      if (in_ != staged_chunk) {
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        const int total = nrows * args.gpr;
        for (int i = etid; i < total; i += EPI_WARPS * 32) {
          const int n = i / args.gpr, g = i - n * args.gpr;
          scaleT[g * SCALE_PITCH + n] = __ldg(args.scale + (size_t)(row0 + n) * args.gpr + g);
        }
        if (!(ok = role_sync(epi_sync_bar, sync_count, 10))) break;
        staged_chunk = in_;
      }
      float running[MY_COLS];
#pragma unroll
      for (int c = 0; c < MY_COLS; ++c) running[c] = 0.f;
      const bool live = n_loc < nrows;
      const int n_safe = live ? n_loc : 0;
      const int pbase = (it - item_begin) * periods_per_item;
      for (int pi = 0; pi < periods_per_item && ok; ++pi) {
        const int pd = pbase + pi, acc = pd & 1;
        if (lane == 0) ok = ptx::mbar_wait_bounded(acc_full(acc), ((uint32_t)(pd >> 1)) & 1u, abort_flag, 8, WAIT_NS);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * args.n_mma) +
                                (FEW ? 0u : (uint32_t)(chalf * MY_COLS));
        const int g0 = pi * args.G;
        if (FEW) {
          uint32_t r[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) r[c] = 0u;
          if (active_warp) {
            ptx::tmem_ld_32x32b_x16(t_addr, r);
            ptx::tmem_ld_wait_16(r);
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(acc_empty(acc));
          if (active_warp) {
            // column c = g_local * mtok + token; running[] stays indexed by column so that every index is a constant
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              int g = g0 + (c >> mtok_shift);
              if (g >= args.gpr) g = args.gpr - 1;   // columns of groups past K hold zeros
              const float s = __uint_as_float((uint32_t)scaleT[g * SCALE_PITCH + n_safe] << 16);
              running[c] = fmaf(s, __uint_as_float(r[c]), running[c]);
            }
          }
        } else {
          const float s = __uint_as_float((uint32_t)scaleT[min(g0, args.gpr - 1) * SCALE_PITCH + n_safe] << 16);
#pragma unroll
          for (int c0 = 0; c0 < MY_COLS; c0 += 16) {
            uint32_t r[16];
            ptx::tmem_ld_32x32b_x16(t_addr + (uint32_t)c0, r);
            ptx::tmem_ld_wait_16(r);
#pragma unroll
            for (int c = 0; c < 16; ++c) running[c0 + c] = fmaf(s, __uint_as_float(r[c]), running[c0 + c]);
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(acc_empty(acc));
        }
      }
      if (!ok) break;
      // ---- store: y[m][row0 + n_loc] = bf16(sum + bias)
      if (live && active_warp) {
        const int n = row0 + n_loc;
        const float b = args.bias ? args.bias[n] : 0.f;
        if (FEW) {
          // fold the G group slots of each token: column c holds token c & (mtok - 1)
#pragma unroll
          for (int m = 0; m < 16; ++m) {
            if (m < mtok && m < args.M) {
              float v = 0.f;
#pragma unroll
              for (int c = 0; c < 16; ++c)
                if ((c & (mtok - 1)) == m) v += running[c];
              args.y[(size_t)m * args.N + n] = __bfloat16_as_ushort(__float2bfloat16_rn(v + b));
            }
          }
        } else {
          const int m0 = im * MT_LARGE + chalf * MY_COLS;
#pragma unroll
          for (int c = 0; c < MY_COLS; ++c) {
            const int m = m0 + c;
            if (m < args.M) args.y[(size_t)m * args.N + n] = __bfloat16_as_ushort(__float2bfloat16_rn(running[c] + b));
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
    ptx::tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && args.status != nullptr) atomicCAS(args.status, 0, *abort_flag);
}

template <int MT_LARGE>
int launch_umma(const CUtensorMap& tw, const CUtensorMap& tx, const UmmaArgs& a, int grid, cudaStream_t stream) {
  const int smem = Smem<MT_LARGE>::total(a.raw_stages, a.op_stages, a.gpr);
  auto kfn = a16_w4_umma_kernel<MT_LARGE>;
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

}  // namespace

int a16_w4_umma_supported(long long M, int N, int K, int group, const char** why) {
  const char* w = nullptr;
  if (M < 1 || M > 0x7fffffffLL) w = "M out of range";
  else if (N < 1) w = "empty N";
  else if (K % KB != 0) w = "K must be a multiple of 64";
  else if (group < KB || group % KB != 0 || K % group != 0) w = "the group size must be a multiple of 64 that divides K";
  else if ((K / 2) % 16 != 0) w = "the weight row pitch must be a multiple of 16 bytes";
  else if (Smem<128>::total(2, 2, K / group) > 227 * 1024) w = "the scales and zero points of one 128-row tile do not fit in shared memory";
  if (why) *why = w;
  return w == nullptr;
}

int a16_w4_umma_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       long long M, int N, int K, int group, int* status, cudaStream_t stream) {
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
  const bool few = M <= 16;
  int mt_large = 0;
  if (few) {
    a.mtok = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
    a.G = 16 / a.mtok;
    a.n_mma = 16;
    a.items_m = 1;
  } else {
    mt_large = M <= 32 ? 32 : M <= 64 ? 64 : 128;
    a.mtok = mt_large;
    a.G = 1;
    a.n_mma = mt_large;
    a.items_m = (int)((M + mt_large - 1) / mt_large);
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
  a.idesc = ptx::make_idesc(1u, 1u, 1u, (uint32_t)TILE_ROWS, (uint32_t)a.n_mma);
  const long long items = (long long)a.items_n * a.items_m;
  const int grid = (int)(items < sms ? items : sms);

  // ring depths: as deep as shared memory allows next to the scales and zero points (at most 4 raw stages of 256 k,
  // at most 6 k-blocks of operands)
  a.raw_stages = 4;
  a.op_stages = few ? 6 : 4;
  auto fits = [&](int rs, int os) {
    const int t = few ? Smem<0>::total(rs, os, a.gpr)
                      : mt_large == 32 ? Smem<32>::total(rs, os, a.gpr)
                                       : mt_large == 64 ? Smem<64>::total(rs, os, a.gpr) : Smem<128>::total(rs, os, a.gpr);
    return t <= 227 * 1024;
  };
  while (!fits(a.raw_stages, a.op_stages)) {
    if (a.op_stages > 4) --a.op_stages;
    else if (a.raw_stages > 2) --a.raw_stages;
    else if (a.op_stages > 2) --a.op_stages;
    else return set_error(B200Q_ERR_UNSUPPORTED, "a16 w4 tensor-core kernel: shared memory does not hold two stages");
  }

  CUtensorMap tw, tx;
  {
    const uint64_t dims[2] = {(uint64_t)(K / 2), (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)(K / 2)};
    const uint32_t box[2] = {128u, 16u};
    B200Q_TRY(make_tmap_u8(&tw, wq, 2, dims, strides, box));
  }
  if (few) {
    tx = tw;  // not used by the few-token form
    return launch_umma<0>(tw, tx, a, grid, stream);
  }
  {
    const uint64_t dims[2] = {(uint64_t)K * 2, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {128u, (uint32_t)mt_large};
    B200Q_TRY(make_tmap_u8(&tx, x, 2, dims, strides, box));
  }
  if (mt_large == 32) return launch_umma<32>(tw, tx, a, grid, stream);
  if (mt_large == 64) return launch_umma<64>(tw, tx, a, grid, stream);
  return launch_umma<128>(tw, tx, a, grid, stream);
}

}  // namespace b200q
