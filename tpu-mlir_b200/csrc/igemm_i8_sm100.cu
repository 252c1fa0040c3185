// INT8 GEMM / implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05 kind::i8).
//
// One persistent CTA per SM walks output tiles of 128 rows x BLOCK_N channels.  Warp roles:
//   warp 0      TMA producer: 128-byte-swizzled K-major tiles of A (activations) and B (weights) into a
//               shared-memory ring, completion counted on mbarriers;
//   warp 1      allocates TMEM and issues tcgen05.mma (one thread), int32 accumulators live in TMEM,
//               two accumulator buffers so the next tile's MMAs overlap this tile's epilogue;
//   warps 2..17 epilogue (one warp per 32 TMEM lanes x BLOCK_N/4 columns): tcgen05.ld the accumulator, + bias, ReLU, exact requantisation
//               (requant.cuh), saturate, store as [rows, N], as NCHW, or as zero-bordered NHWC.
//
// The convolution is expressed as a GEMM whose A rows are the pixels of a zero-bordered NHWC image
// flattened to [N*Hp*Wp, C]: the row block of filter tap (fy, fx) is the same row block shifted by
// (fy - pad_top) * Wp + (fx - pad_left) rows, so every A tile is still one 2-D TMA box (rows outside the
// tensor are zero-filled by TMA).  Outputs computed for border pixels are discarded (or written as zero).
// This replaces tpu::MatMulOp / tpu::Conv2DOp inference (lib/Dialect/Tpu/Interfaces/Common/MatMul.cpp:599-728,
// Conv2D.cpp:264-341) and the oneDNN primitives behind them (lib/Support/Dnnl/MatMul.cpp, Conv.cpp).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdlib.h>

#include "igemm.h"
#include "internal.h"
#include "ptx_sm100.cuh"
#include "round16.cuh"
#include <atomic>
#include <cmath>

#include "requant.cuh"

namespace b200q {

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;  // bytes == int8 elements: one 128-byte swizzle span
constexpr int KIND_BF16_TAG = -2;  // value of the DIALECT template argument that selects bf16 operands / output  // each epilogue warp owns 32 TMEM lanes x 64 columns of the tile
constexpr uint64_t DEFAULT_WAIT_BUDGET_NS = 2000000000ull;  // 2 s: far above any legitimate tile time

// PAIR: two CTAs of a cluster compute one 256 x BLOCK_N tile with tcgen05 cta_group::2; each CTA stages its own 128
// rows of A and half of B's N rows, so a CTA pulls 1.5x fewer operand bytes per MMA through L2 and shared memory.
// TAPW = 3: the three taps of a filter row share ONE activation block of 128 + 2 rows per stage (tap fx starts fx
// rows into it), next to the three taps' weight tiles: a third of the activation traffic per MMA.
template <int BLOCK_N, int STAGES, bool PAIR = false, int TAPW = 1>
struct SmemLayout {
  static constexpr int A_ROWS = BLOCK_M + (TAPW - 1);
  static constexpr int A_BOX_BYTES = A_ROWS * BLOCK_K;                 // what the TMA box delivers
  static constexpr int A_BYTES = (A_BOX_BYTES + 1023) & ~1023;         // B tiles stay 1024-byte aligned
  static constexpr int B_ROWS = PAIR ? BLOCK_N / 2 : BLOCK_N;  // rows of B this CTA stages
  static constexpr int B_BYTES = B_ROWS * BLOCK_K;
  static constexpr int STAGE_BYTES = A_BYTES + TAPW * B_BYTES;
  static constexpr int STAGE_TX = A_BOX_BYTES + TAPW * B_BYTES;        // bytes one CTA's loads deliver per stage
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;  // tmem ptr, abort flag
  static constexpr int CHAN_OFFSET = MISC_OFFSET + 16;           // {bias, multiplier, shift, -} of the tile's channels
  static constexpr int SLOW_OFFSET = CHAN_OFFSET + BLOCK_N * 16;  // per 32-channel chunk: the staged parameter form
  static constexpr int CHANK_OFFSET = SLOW_OFFSET + (BLOCK_N / 32) * 4;  // folded form: rounding constant + shifted zero point
  static constexpr int RES_OFFSET = (CHANK_OFFSET + BLOCK_N * 4 + 15) & ~15;  // fused Add: 512 bytes of scratch per epilogue warp
  static constexpr int TOTAL = RES_OFFSET + 16 * 512;
  static constexpr int DYN_BYTES = TOTAL + 1024;                 // slack for manual 1024-byte alignment
  // always 16 epilogue warps (4 TMEM lane quarters x 4 column groups): a narrow tile is split finer instead of
  // leaving warps idle, its epilogue costs as much per element as a wide one's
  static constexpr int EPI_WARPS = 16;
  static constexpr int EPI_COLS = BLOCK_N / 4;  // columns per epilogue warp: 64, 32 or 16
  static constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
  // 18 warps land 5,5,4,4 on the four sub-partitions (16384 registers each): 96 registers per thread at most
};

template <int BLOCK_N>
struct TmemCols {
  static constexpr int value = (2 * BLOCK_N) < 32 ? 32 : 2 * BLOCK_N;  // power of two for BLOCK_N in {16,...,256}
};

// how a 32-channel chunk's requantisation parameters are staged (see the epilogue)
enum { FORM_FOLD_QDM = 0, FORM_FAST = 1, FORM_GENERAL = 3, FORM_FOLD_HI = 4, FORM_FOLD_FUNNEL = 5 };

// Tile index -> (row tile, column tile).  Tiles are walked in bands of `band_m` row tiles, column tile by column tile
// inside a band, so that the tiles in flight at any moment (consecutive indices: the workers stride by their count)
// form a roughly square block and share their operand rows in L2 instead of sweeping all of B once per row of tiles.
__device__ __forceinline__ void tile_coords(const IGemmArgs& args, int tile, int& mt, int& nt) {
  if (args.band_m <= 1) {
    mt = tile / args.num_n_tiles;
    nt = tile - mt * args.num_n_tiles;
    return;
  }
  const int per_band = args.band_m * args.num_n_tiles;
  const int band = tile / per_band;
  const int idx = tile - band * per_band;
  const int m_first = band * args.band_m;
  const int height = min(args.band_m, args.num_m_tiles - m_first);
  nt = idx / height;
  mt = m_first + (idx - nt * height);
}

template <int THREADS>
__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}


__device__ __forceinline__ int32_t add_sat_s32(int32_t a, int32_t b) {
  int32_t r;
  asm("add.sat.s32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Fast requantisation cores for the two forms real graphs use.  They are exact restatements of
// requant_value<> restricted to a parameter domain that is checked per channel when the channel
// parameters are staged in shared memory (anything outside takes the general path):
//   QDM, half away from zero:   multiplier != INT32_MIN, right shift t in [1,31]   (p0 = t, p1 = 2^(t-1))
//   MultiplierShift, half up:   right shift s in [1,62]                            (p0 = s)
// Both return a value clamped to int32; zero point, ReLU and the output saturation follow in 32 bits.
template <int DIALECT>
__device__ __forceinline__ int32_t requant_core_fast(int32_t a, int32_t m, int32_t p0, int32_t p1) {
  if (DIALECT == B200Q_RQ_QDM) {
    const int64_t x = ptx::mad_wide_s32(a, m, 1ll << 30);  // floor((a*m + 2^30) / 2^31) == half-up shift by 31
    const int32_t v = (int32_t)(x >> 31);                     // |a*m| <= 2^62 - 2^31: always fits int32 here
    const int32_t mant = v & ((p1 << 1) - 1);
    const int32_t ge0 = (int32_t)((uint32_t)(~v) >> 31);
    return (v >> p0) + (int32_t)((mant + ge0) > p1);
  } else {
    int64_t x = ptx::mad_wide_s32(a, m, (int64_t)(1ull << (p0 - 1))) >> p0;
    return x > 2147483647ll ? 2147483647 : (x < -2147483648ll ? (int32_t)(-2147483647 - 1) : (int32_t)x);
  }
}

template <int DIALECT, int RMODE>
__device__ __forceinline__ bool fast_domain(int32_t m, int32_t s) {
  if (DIALECT == B200Q_RQ_QDM && RMODE == B200Q_ROUND_HALF_AWAY_FROM_ZERO) return m != (-2147483647 - 1) && s <= -1 && s >= -31;
  if (DIALECT == B200Q_RQ_MULTIPLIER_SHIFT && RMODE == B200Q_ROUND_HALF_UP) return s >= 1 && s <= 62;
  return false;
}

// Extra conditions of the folded forms (on top of fast_domain, |bias| < 2^28 and |accumulator| < 2^29), chosen so
// that no 64-bit intermediate can overflow: QDM: |zp| << t < 2^28;  MultiplierShift: |zp| << s < 2^60 (the epilogue
// additionally proves that a value shifted by s < 32 fits 32 bits).
template <int DIALECT>
__device__ __forceinline__ bool fold_domain(int32_t sh, int32_t zp) {
  const long long az = zp < 0 ? -(long long)zp : (long long)zp;
  if (DIALECT == B200Q_RQ_QDM) return az < (1ll << 20) && (az << (-sh)) < (1ll << 28);
  if (DIALECT == B200Q_RQ_MULTIPLIER_SHIFT) return sh >= 1 && sh <= 62 && az < (1ll << 20) && (zp == 0 || sh <= 40);
  return false;
}


// Classification of one output channel's parameters: bit 1 = not foldable, 2 = not in the fast domain,
// 4 = foldable MultiplierShift with s in [1,31] (funnel form), 8 = foldable MultiplierShift with s >= 32.
template <int DIALECT, int RMODE>
__device__ __forceinline__ int classify_channel(int32_t bias, int32_t m, int32_t sh, const IGemmArgs& args, bool fast_dialect) {
  const Epilogue& e = args.epi;
  const bool pre_relu = e.relu == B200Q_RELU_BEFORE_REQUANT;
  const long long az = e.out_zp < 0 ? -(long long)e.out_zp : (long long)e.out_zp;
  const bool fast_ok = fast_dialect && fast_domain<DIALECT, RMODE>(m, sh);
  bool fold_ok = fast_ok && !pre_relu && args.acc_small && bias > -(1 << 28) && bias < (1 << 28) &&
                 fold_domain<DIALECT>(sh, e.out_zp);
  int width_bits = 0;
  if (DIALECT == B200Q_RQ_MULTIPLIER_SHIFT && fold_ok) {
    if (sh >= 32) {
      width_bits = 8;
    } else {  // the value shifted by s must fit 32 bits for every accumulator this K can produce
      const unsigned long long am = (unsigned long long)(m < 0 ? -(long long)m : (long long)m);
      const unsigned long long ab = (unsigned long long)(bias < 0 ? -(long long)bias : (long long)bias);
      const unsigned long long bound = (unsigned long long)args.acc_bound * am + ab * am + (1ull << (sh - 1)) +
                                       ((unsigned long long)az << sh);
      fold_ok = bound < (1ull << (31 + sh));
      width_bits = 4;
    }
  }
  return (fold_ok ? width_bits : 1) | (fast_ok ? 0 : 2);
}

// The cheapest form every channel of a group allows, from the OR of the group's classification bits.
template <int DIALECT>
__device__ __forceinline__ int form_of_bits(int st, bool relu_after) {
  if (st & 2) return FORM_GENERAL;
  if (st & 1) return FORM_FAST;
  if (DIALECT == B200Q_RQ_QDM) return relu_after ? FORM_FOLD_HI : FORM_FOLD_QDM;
  return ((st & 4) && (st & 8)) ? FORM_FAST : ((st & 4) ? FORM_FOLD_FUNNEL : FORM_FOLD_HI);
}

// One channel's constants in the layout `form` reads (see the table in the kernel); `in` false: a channel past N.
template <int DIALECT>
__device__ __forceinline__ void form_constants(int form, bool in, int32_t bias, int32_t m, int32_t sh, int32_t out_zp,
                                               int4* cp, int32_t* ck) {
  *ck = 0;
  if (!in) {
    *cp = make_int4(0, 0, 0, 1);
  } else if (form == FORM_FOLD_HI || form == FORM_FOLD_FUNNEL || form == FORM_FOLD_QDM) {
    long long C;
    int32_t s4;
    if (DIALECT == B200Q_RQ_QDM) {
      const int32_t t = -sh;
      const long long K = (long long)((1u << t) >> 1) + (long long)((unsigned long long)(long long)out_zp << t);
      C = (long long)bias * (long long)m + (1ll << 30);
      if (form == FORM_FOLD_HI) {
        C += (long long)((unsigned long long)K << 31);
        s4 = t - 1;
      } else {  // (w - (w < 0) + K) >> t after w = (acc*m + C) >> 31
        *ck = (int32_t)K;
        s4 = t;
      }
    } else {
      C = (long long)bias * (long long)m + (long long)(1ull << (sh - 1)) + (long long)((unsigned long long)(long long)out_zp << sh);
      s4 = form == FORM_FOLD_HI ? sh - 32 : sh;
    }
    *cp = make_int4((int32_t)(uint32_t)(C & 0xffffffffll), (int32_t)(C >> 32), m, s4);  // C: an aligned register pair
  } else if (form == FORM_FAST) {
    const int32_t t = DIALECT == B200Q_RQ_QDM ? -sh : sh;
    *cp = make_int4(bias, m, t, DIALECT == B200Q_RQ_QDM ? (int32_t)(1u << (t - 1)) : 0);
  } else {
    *cp = make_int4(bias, m, sh, 0);
  }
}

// PERROW: the requantisation parameters belong to the GEMM's ROWS (the transposed product: rows are output channels,
// columns pixels).  Every epilogue thread then keeps its own row's constants in registers; no shared-memory
// parameter read is left in the per-element path, whose 16 bytes per lane and element otherwise saturate the
// load/store pipe of a short-K product.
template <int BLOCK_N, int STAGES, int DIALECT, int RMODE, bool PAIR, int TAPW, bool PERROW = false, bool ADD = false>
__global__ void __launch_bounds__(SmemLayout<BLOCK_N, STAGES, PAIR, TAPW>::NUM_THREADS, 1)
igemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const IGemmArgs args) {
  using L = SmemLayout<BLOCK_N, STAGES, PAIR, TAPW>;
  static_assert(TAPW == 1 || PAIR, "the tap-fused form exists for CTA pairs only");
  ptx::griddep_launch_dependents();  // a dependent kernel may become resident as this grid's CTAs retire
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFFSET + 4);
  int4* chan = reinterpret_cast<int4*>(smem + L::CHAN_OFFSET);
  int* chunk_form = reinterpret_cast<int*>(smem + L::SLOW_OFFSET);
  int32_t* chan_k = reinterpret_cast<int32_t*>(smem + L::CHANK_OFFSET);
  constexpr int EPI_THREADS = L::EPI_WARPS * 32;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // PAIR: CTA 0 of the cluster leads (expects the bytes of both CTAs' loads, issues the MMAs); a worker is a CTA pair
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), PAIR ? 2 * L::EPI_WARPS : EPI_THREADS);  // PAIR: one arrival per warp, both CTAs
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (PAIR) {
    __syncthreads();
    ptx::cluster_sync_all();  // the peer's barriers exist before anything can signal them
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(tmem_ptr_smem), TmemCols<BLOCK_N>::value);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), TmemCols<BLOCK_N>::value);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_tiles = args.num_m_tiles * args.num_n_tiles;
  const int num_kb = args.num_kb;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      ptx::griddep_wait();  // the operands may be the previous kernel's output (the set-up above overlapped its tail)
      for (int tile = worker; tile < num_tiles && ok; tile += num_workers) {
        int mt, nt;
        tile_coords(args, tile, mt, nt);
        const int m0 = mt * TILE_M + (int)cta_rank * BLOCK_M;
        const int n0 = nt * BLOCK_N;
        // k-block inside the tap and the tap's row shift are counted, not divided: this loop is serial
        int kc = 0, fx = 0;
        int a_row = m0 - args.tap_org_h * args.row_pitch - args.tap_org_w;  // tap (0,0)
        if (TAPW > 1) {
          // one stage = the three taps of filter row fy at k-block kc: one 130-row activation block, three weight tiles
          const int groups = num_kb / TAPW;
          int fy = 0;
          for (int g = 0; g < groups; ++g) {
            ok = ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, 1, args.wait_budget_ns);
            if (!ok) break;
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_TX + args.expect_extra);
            const uint32_t lead_bar = ptx::map_to_cta(full_bar(stage), 0);
            ptx::tma_load_2d_pair(sa, &tmap_a, lead_bar, kc * BLOCK_K, a_row);
#pragma unroll
            for (int t = 0; t < TAPW; ++t)
              ptx::tma_load_2d_pair(sa + L::A_BYTES + t * L::B_BYTES, &tmap_b, lead_bar,
                                    ((fy * TAPW + t) * args.kb_per_tap + kc) * BLOCK_K, n0 + (int)cta_rank * L::B_ROWS);
            if (++kc == args.kb_per_tap) {
              kc = 0;
              ++fy;
              a_row += args.row_pitch;
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        } else {
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, 1, args.wait_budget_ns);
          if (!ok) break;
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          if (PAIR) {
            // both CTAs' bytes complete on the leader's barrier; only the leader arrives on it
            if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES + args.expect_extra);
            const uint32_t lead_bar = ptx::map_to_cta(full_bar(stage), 0);
            ptx::tma_load_2d_pair(sa, &tmap_a, lead_bar, kc * BLOCK_K, a_row);
            ptx::tma_load_2d_pair(sa + L::A_BYTES, &tmap_b, lead_bar, kb * BLOCK_K, n0 + (int)cta_rank * L::B_ROWS);
          } else {
            ptx::mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES + args.expect_extra);
            ptx::tma_load_2d(sa, &tmap_a, full_bar(stage), kc * BLOCK_K, a_row);
            ptx::tma_load_2d(sa + L::A_BYTES, &tmap_b, full_bar(stage), kb * BLOCK_K, n0);
          }
          if (++kc == args.kb_per_tap) {
            kc = 0;
            a_row += args.tap_step_w;  // next tap of the filter row
            if (++fx == args.taps_w) {
              fx = 0;
              a_row += args.row_pitch - args.taps_w * args.tap_step_w;  // first tap of the next filter row
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // K-major, 128-byte swizzle, 8-row groups 1024 bytes apart: only the start address differs between tiles
      const uint64_t desc0 = ptx::make_smem_desc_kmajor(smem_base, 1024, 2);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)desc0;
      const uint32_t b_lo0 = (uint32_t)ptx::make_smem_desc_kmajor(smem_base + L::A_BYTES, 1024, 2);
      for (int tile = worker; tile < num_tiles && ok; tile += num_workers) {
        ok = ptx::mbar_wait_bounded(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, 2, args.wait_budget_ns);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
        for (int kb = 0; kb < num_kb / TAPW; ++kb) {
          ok = ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, 3, args.wait_budget_ns);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t so = (uint32_t)stage * (uint32_t)(L::STAGE_BYTES >> 4);  // descriptor address units of 16 bytes
          const uint32_t accum = kb != 0 ? 1u : 0u;
          if (TAPW > 1) {
#pragma unroll
            for (int t = 0; t < TAPW; ++t) {
              // tap t reads the activation block from row t on: only the start address moves.  The 128-byte swizzle is
              // a function of the shared-memory address bits, which TMA used when it wrote the block, so no
              // base-offset correction is needed (measured: setting the descriptor's base-offset field breaks it).
              const uint32_t al = a_lo0 + so + (uint32_t)(t * (BLOCK_K >> 4));
              const uint32_t bl = b_lo0 + so + (uint32_t)(t * (L::B_BYTES >> 4));
              if (DIALECT == KIND_BF16_TAG) ptx::umma_kblock_f16_pair(d_tmem, al, bl, desc_hi, desc_hi, args.idesc, (t | (int)accum) != 0 ? 1u : 0u);
              else ptx::umma_kblock_i8_pair(d_tmem, al, bl, desc_hi, desc_hi, args.idesc, (t | (int)accum) != 0 ? 1u : 0u);
            }
          } else if (PAIR) {
            if (DIALECT == KIND_BF16_TAG) ptx::umma_kblock_f16_pair(d_tmem, a_lo0 + so, b_lo0 + so, desc_hi, desc_hi, args.idesc, accum);
            else ptx::umma_kblock_i8_pair(d_tmem, a_lo0 + so, b_lo0 + so, desc_hi, desc_hi, args.idesc, accum);
          } else {
            if (DIALECT == KIND_BF16_TAG) ptx::umma_kblock_f16(d_tmem, a_lo0 + so, b_lo0 + so, desc_hi, desc_hi, args.idesc, accum);
            else ptx::umma_kblock_i8(d_tmem, a_lo0 + so, b_lo0 + so, desc_hi, desc_hi, args.idesc, accum);
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) ptx::umma_commit_pair(empty_bar(stage), 3);
          else ptx::umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (PAIR) ptx::umma_commit_pair(tmem_full_bar(acc), 3);  // accumulator complete (each CTA holds its 128 rows)
        else ptx::umma_commit(tmem_full_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;                                   // TMEM lanes 32*quarter .. 32*quarter+31
    const int col0 = ((warp - 2) >> 2) * L::EPI_COLS;               // first tile column of this warp
    const int etid = threadIdx.x - 64;
    const Epilogue& e = args.epi;
    const bool out8 = e.out_dtype == B200Q_DT_I8 || e.out_dtype == B200Q_DT_U8;
    // the fast cores need an output type whose range lies inside int32 after the zero point is added
    constexpr bool kFastCompiled = (DIALECT == B200Q_RQ_QDM && RMODE == B200Q_ROUND_HALF_AWAY_FROM_ZERO) ||
                                   (DIALECT == B200Q_RQ_MULTIPLIER_SHIFT && RMODE == B200Q_ROUND_HALF_UP);
    const bool kFastDialect = kFastCompiled && e.out_dtype != B200Q_DT_I32;
    const int32_t zp = e.out_zp;
    // The output range, the ReLU floors and the flags derived from them are kernel parameters (the host fills them in):
    // as constant-bank operands they hold no registers across the tile loop.
    //   sat_lo2 = max(type minimum, post-ReLU floor): clamp(max(v, f), lo, hi) == clamp(v, max(lo, f), hi) for f <= hi
    //   pack_sat: rows of packed bytes leave the clamping to the saturating pack (plus one max when floor_needed, i.e.
    //   a post-ReLU floor lies above the type's lowest value)
    const bool relu_after = e.relu == B200Q_RELU_AFTER_REQUANT;
#define floor_pre (args.floor_pre)
#define sat_lo2 (args.sat_lo2)
#define sat_hi (args.sat_hi)
#define pack_sat (args.pack_sat != 0)
#define floor_needed (args.floor_needed != 0)
    ptx::griddep_wait();  // before the first read of a parameter array or write of the output
    int acc = 0;
    uint32_t acc_phase = 0;
    int cached_n0 = -1;
    int row_form = FORM_GENERAL;  // PERROW: this thread's row
    int4 row_cp = make_int4(0, 0, 0, 1);
    int32_t row_ck = 0;
    const uint32_t lead_tmem_empty0 = PAIR ? ptx::map_to_cta(tmem_empty_bar(0), 0) : 0u;
    for (int tile = worker; tile < num_tiles; tile += num_workers) {
      int mt, nt;
      tile_coords(args, tile, mt, nt);
      const int m0 = mt * TILE_M + (int)cta_rank * BLOCK_M;
      const int n0 = nt * BLOCK_N;
      if (PERROW) {
        if (m0 != cached_n0) {  // (cached_n0 holds the row tile here) the constants of this thread's row
          const int ch = m0 + quarter * 32 + lane;
          const bool in = ch < args.rows;
          const int32_t bias = (in && e.bias) ? e.bias[ch] : 0;
          const int32_t m = (in && e.multiplier) ? e.multiplier[e.per_channel ? ch : 0] : 1;
          const int32_t sh = (in && e.shift) ? e.shift[e.per_channel ? ch : 0] : 0;
          const int bits = in ? classify_channel<DIALECT, RMODE>(bias, m, sh, args, kFastDialect) : 0;
          row_form = form_of_bits<DIALECT>((int)__reduce_or_sync(0xffffffffu, (unsigned)bits), relu_after);  // one form per warp
          form_constants<DIALECT>(row_form, in, bias, m, sh, e.out_zp, &row_cp, &row_ck);
          cached_n0 = m0;
        }
      } else if (n0 != cached_n0) {
        // Stage the tile's channel parameters in the cheapest form every channel of a 32-channel chunk allows:
        //   FOLD_HI     {m, C_lo, C_hi, sh}: v = hi32(acc*m + C) >> sh.  Bias, every rounding constant and the zero
        //               point live in C.  QDM with the ReLU after the requantisation (the sign term of the second,
        //               half-away rounding only matters for results the ReLU clamps anyway): C = bias*m + 2^30 +
        //               (2^(t-1) + (zp << t)) * 2^31, sh = t - 1.  MultiplierShift with s >= 32: sh = s - 32.
        //   FOLD_FUNNEL MultiplierShift with s in [1,31] whose shifted value provably fits 32 bits:
        //               v = low32((acc*m + C) >> s), C = bias*m + 2^(s-1) + (zp << s).
        //   FOLD_QDM    {m, C_lo, C_hi, t} + chan_k: QDM half-away without the ReLU shortcut.
        //   FAST        {bias, m, right shift, half}: the pre-ReLU (MatMul) order, or biases too large to fold
        //   GENERAL     {bias, m, shift, 0}: any dialect / rounding mode / parameter value (requant_value<>)
        epi_bar_sync<EPI_THREADS>();  // everyone is done reading the previous tile's channel parameters
        if (etid < BLOCK_N / 32) chunk_form[etid] = 0;
        epi_bar_sync<EPI_THREADS>();
        for (int c = etid; c < BLOCK_N; c += EPI_THREADS) {
          if (DIALECT == KIND_BF16_TAG) break;
          const int n = n0 + c;
          if (n >= args.n) continue;
          const int32_t bias = e.bias ? e.bias[n] : 0;
          const int32_t m = e.multiplier ? e.multiplier[e.per_channel ? n : 0] : 1;
          const int32_t sh = e.shift ? e.shift[e.per_channel ? n : 0] : 0;
          atomicOr(&chunk_form[c >> 5], classify_channel<DIALECT, RMODE>(bias, m, sh, args, kFastDialect));
        }
        epi_bar_sync<EPI_THREADS>();
        int my_form[(BLOCK_N + EPI_THREADS - 1) / EPI_THREADS];
#pragma unroll
        for (int i = 0; i < (BLOCK_N + EPI_THREADS - 1) / EPI_THREADS; ++i) {
          const int c = etid + i * EPI_THREADS;
          if (c >= BLOCK_N) break;
          const int n = n0 + c;
          const bool in = n < args.n;
          if (DIALECT == KIND_BF16_TAG) {
            chan[c] = make_int4((in && args.bias_f32) ? __float_as_int(args.bias_f32[n]) : 0, 0, 0, 0);
            my_form[i] = FORM_GENERAL;
            continue;
          }
          const int32_t bias = (in && e.bias) ? e.bias[n] : 0;
          const int32_t m = (in && e.multiplier) ? e.multiplier[e.per_channel ? n : 0] : 1;
          const int32_t sh = (in && e.shift) ? e.shift[e.per_channel ? n : 0] : 0;
          const int form = form_of_bits<DIALECT>(chunk_form[c >> 5], relu_after);
          my_form[i] = form;
          int4 cp;
          int32_t ck;
          form_constants<DIALECT>(form, in, bias, m, sh, e.out_zp, &cp, &ck);
          chan[c] = cp;
          chan_k[c] = ck;
        }
        epi_bar_sync<EPI_THREADS>();  // every thread has read its chunks' classification bits
        if (DIALECT != KIND_BF16_TAG) {
#pragma unroll
          for (int i = 0; i < (BLOCK_N + EPI_THREADS - 1) / EPI_THREADS; ++i) {
            const int c = etid + i * EPI_THREADS;
            if (c < BLOCK_N && (c & 31) == 0) chunk_form[c >> 5] = my_form[i];
          }
        }
        epi_bar_sync<EPI_THREADS>();
        cached_n0 = n0;
      }
      const int row = m0 + quarter * 32 + lane;
      // where this row goes
      bool row_valid = row < args.rows;
      bool write_zero_row = false;
      long long out_base = 0;  // element offset of (row, channel 0)
      int chan_stride = 1;
      if (args.out_mode == IGEMM_OUT_ROWMAJOR) {
        out_base = (long long)row * args.ldc;
      } else {
        const int img = row / args.img_rows;
        const int rem = row - img * args.img_rows;
        const int hp = rem / args.row_pitch;
        const int wp = rem - hp * args.row_pitch;
        const int h = hp - args.border_h, w = wp - args.border_w;
        const bool interior = row_valid && h >= 0 && h < args.out_h && w >= 0 && w < args.out_w;
        if (args.out_mode == IGEMM_OUT_NCHW) {
          row_valid = interior;
          out_base = ((long long)img * args.n * args.out_h + h) * args.out_w + w;
          chan_stride = args.out_h * args.out_w;
        } else if (args.out_mode == IGEMM_OUT_NHWC) {  // unbordered NHWC: border rows are dropped
          row_valid = interior;
          out_base = (((long long)img * args.out_h + h) * args.out_w + w) * args.ldc;
        } else {  // zero-bordered NHWC: border rows are written as zeros
          out_base = (long long)row * args.ldc;
          write_zero_row = row_valid && !interior;
          row_valid = interior;
        }
      }

      // 16 columns per TMEM load keep the epilogue's live registers low.  The read is not overlapped with the previous
      // chunk's arithmetic inside a warp (a second register set costs more in spills and lost instruction-level
      // parallelism than the read's latency, which the other warps of the scheduler cover).
      constexpr int CH = 16;
      const uint32_t t_warp = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N + col0);
      // Fused residual Add: the other operand's 16 bytes of a chunk, packed four to a register, requested one chunk
      // ahead (the first before the wait for the accumulator) so that their latency hides behind the tensor-memory
      // read and the requantisation of the chunk before.
      // Transposed product (rows = channels): a chunk's residual bytes are 16 pixels x this warp's 32 channels, 32
      // contiguous bytes per pixel.  Lane i fetches the 16-byte piece i (pixel i / 2, half i % 2) with one load; when
      // the chunk is processed the pieces go through 512 bytes of warp-private shared memory, from which every lane
      // reads its own channel's byte of each pixel.
      const bool res_vec = ADD && PERROW && ((reinterpret_cast<uintptr_t>(args.res) & 15) == 0) && (chan_stride & 15) == 0;
      uint8_t* const res_sm = smem + L::RES_OFFSET + (warp - 2) * 512;
      auto load_res = [&](int cc_, uint32_t (&rw)[CH / 4]) {
#pragma unroll
        for (int w = 0; w < CH / 4; ++w) rw[w] = 0u;
        const int cb = col0 + cc_ * CH;
        const int nc = min(CH, args.n - (n0 + cb));
        if (res_vec) {
          if ((lane >> 1) < nc) {
            const uint8_t* rp = args.res + (long long)(n0 + cb + (lane >> 1)) * chan_stride + (m0 + quarter * 32) + 16 * (lane & 1);
            const uint4 v4 = __ldg(reinterpret_cast<const uint4*>(rp));
            rw[0] = v4.x, rw[1] = v4.y, rw[2] = v4.z, rw[3] = v4.w;
          }
          return;
        }
        if (!row_valid || nc <= 0) return;
        if (args.out_mode == IGEMM_OUT_NCHW) {
          const uint8_t* rp = args.res + out_base + (long long)(n0 + cb) * chan_stride;
#pragma unroll
          for (int j = 0; j < CH; ++j)
            if (j < nc) rw[j >> 2] |= (uint32_t)__ldg(rp + (long long)j * chan_stride) << (8 * (j & 3));
        } else {
          const uint8_t* rp = args.res + out_base + n0 + cb;
          if (nc == CH && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
            const uint4 v4 = __ldg(reinterpret_cast<const uint4*>(rp));
            rw[0] = v4.x, rw[1] = v4.y, rw[2] = v4.z, rw[3] = v4.w;
          } else {
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (j < nc) rw[j >> 2] |= (uint32_t)__ldg(rp + j) << (8 * (j & 3));
          }
        }
      };
      uint32_t res_next[CH / 4] = {0u, 0u, 0u, 0u};
      if (ADD) load_res(0, res_next);
      if (!ptx::mbar_wait_bounded(tmem_full_bar(acc), acc_phase, abort_flag, 4, args.wait_budget_ns)) break;
      ptx::tc_fence_after_sync();
#pragma unroll 1
      for (int cc = 0; cc < L::EPI_COLS / CH; ++cc) {
        const int cbase = col0 + cc * CH;
        uint32_t res_cur[CH / 4];
#pragma unroll
        for (int w = 0; w < CH / 4; ++w) res_cur[w] = res_next[w];
        if (ADD && cc + 1 < L::EPI_COLS / CH) load_res(cc + 1, res_next);
        uint32_t r[CH];
        ptx::tmem_ld_32x32b_x16(t_warp + (uint32_t)(cc * CH), r);
        ptx::tmem_ld_wait_16(r);
        if (cc == L::EPI_COLS / CH - 1) {
          // this warp's share of the accumulator buffer is in registers: hand it back to the MMA warp.  Nothing
          // written to memory is being published, so the arrival needs no release ordering (which would wait for
          // this thread's earlier global stores).
          ptx::tc_fence_before_sync();
          if (PAIR) {
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster_relaxed(lead_tmem_empty0 + 8u * acc);  // the leader's MMA warp waits on it
          } else {
            ptx::mbar_arrive_relaxed(tmem_empty_bar(acc));
          }
        }
        if (n0 + cbase >= args.n) continue;
        if (DIALECT == KIND_BF16_TAG) {
          // fp32 accumulator (+ bias) -> bf16, row-major [rows, N]
          if (row_valid) {
            const int nc = min(CH, args.n - (n0 + cbase));
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(args.out) + out_base + n0 + cbase;
            uint32_t pk[CH / 2];
#pragma unroll
            for (int j = 0; j < CH / 2; ++j) {
              const float v0 = __uint_as_float(r[2 * j]) + __int_as_float(chan[cbase + 2 * j].x);
              const float v1 = __uint_as_float(r[2 * j + 1]) + __int_as_float(chan[cbase + 2 * j + 1].x);
              if (args.f16) {
                const __half2 h2 = __floats2half2_rn(v0, v1);
                pk[j] = *reinterpret_cast<const uint32_t*>(&h2);
              } else {
                pk[j] = (uint32_t)f32_to_bf16_bits_ref(v0) | ((uint32_t)f32_to_bf16_bits_ref(v1) << 16);
              }
            }
            if (nc == CH && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
              reinterpret_cast<uint4*>(o)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              reinterpret_cast<uint4*>(o)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (j < nc) reinterpret_cast<uint16_t*>(o)[j] = (uint16_t)(pk[j >> 1] >> ((j & 1) * 16));
            }
          }
          continue;
        }
        int32_t q[CH];
        const int form = !kFastCompiled ? FORM_GENERAL : (PERROW ? row_form : chunk_form[cbase >> 5]);
        // packed 8-bit rows: the saturating pack does the clamping, four values per two instructions
        bool raw = false;
        if (kFastCompiled && (form == FORM_FOLD_HI || form == FORM_FOLD_FUNNEL)) {
          if (form == FORM_FOLD_HI) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int4 cp = PERROW ? row_cp : chan[cbase + j];  // {C_lo, C_hi, m, sh}: one broadcast 16-byte shared load
              const long long C = (long long)(((unsigned long long)(uint32_t)cp.y << 32) | (uint32_t)cp.x);
              const long long x = ptx::mad_wide_s32((int32_t)r[j], cp.z, C);
              q[j] = (int32_t)(x >> 32) >> cp.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int4 cp = PERROW ? row_cp : chan[cbase + j];
              const long long C = (long long)(((unsigned long long)(uint32_t)cp.y << 32) | (uint32_t)cp.x);
              const long long x = ptx::mad_wide_s32((int32_t)r[j], cp.z, C);
              q[j] = (int32_t)__funnelshift_r((uint32_t)x, (uint32_t)(x >> 32), (uint32_t)cp.w);
            }
          }
          raw = pack_sat;
          if (!raw) {
            if (sat_lo2 == 0) {  // the usual case after a ReLU: max(min(v, hi), 0) is one instruction
#pragma unroll
              for (int j = 0; j < CH; ++j) q[j] = __vimin_s32_relu(q[j], sat_hi);
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j) q[j] = min(max(q[j], sat_lo2), sat_hi);
            }
          } else if (floor_needed) {
#pragma unroll
            for (int j = 0; j < CH; ++j) q[j] = max(q[j], sat_lo2);
          }
        } else if (kFastCompiled && form == FORM_FOLD_QDM) {
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int4 cp = PERROW ? row_cp : chan[cbase + j];  // {C_lo, C_hi, m, t}
            const long long C = (long long)(((unsigned long long)(uint32_t)cp.y << 32) | (uint32_t)cp.x);
            const long long x = ptx::mad_wide_s32((int32_t)r[j], cp.z, C);
            const int32_t w = (int32_t)(x >> 31);  // half-up shift by 31: C carries the 2^30
            // half away from zero for a right shift by t: (w + 2^(t-1) - (w < 0)) >> t, zero point inside chan_k
            q[j] = min(max((w + (w >> 31) + (PERROW ? row_ck : chan_k[cbase + j])) >> cp.w, sat_lo2), sat_hi);
          }
        } else if (kFastCompiled && form == FORM_FAST) {
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int4 cp = PERROW ? row_cp : chan[cbase + j];  // {bias, multiplier, shift, half}
            const int32_t a = max((int32_t)r[j] + cp.x, floor_pre);
            const int32_t v = requant_core_fast<DIALECT>(a, cp.y, cp.z, cp.w);
            q[j] = min(max(add_sat_s32(v, zp), sat_lo2), sat_hi);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int4 cp = PERROW ? row_cp : chan[cbase + j];  // {bias, multiplier, shift, -}
            int32_t a = (int32_t)r[j] + cp.x;
            if (e.relu == B200Q_RELU_BEFORE_REQUANT && a < 0) a = 0;
            q[j] = requant_value<-1, -1>(a, cp.y, cp.z, e);
          }
        }
        const int ncols = min(CH, args.n - (n0 + cbase));
        if (ADD && res_vec) {   // warp-uniform: every lane of the warp holds one piece
          __syncwarp();         // the previous chunk's bytes have been read
          *reinterpret_cast<uint4*>(res_sm + lane * 16) = make_uint4(res_cur[0], res_cur[1], res_cur[2], res_cur[3]);
          __syncwarp();
        }
        if (ADD && row_valid) {
          // fused residual Add: the product's own output (saturated to its type) and the other operand, each through
          // its multiplier and half-up shift, summed and clamped to the Add's range (its ReLU is the lower bound)
#pragma unroll
          for (int j = 0; j < CH; ++j) q[j] = min(max(q[j], sat_lo2), sat_hi);   // (the packed store would have done it)
          raw = false;
          const int32_t hs = 1 << (args.add_s_self - 1), hr = 1 << (args.add_s_res - 1);
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const uint32_t b = res_vec ? (uint32_t)res_sm[j * 32 + lane] : ((res_cur[j >> 2] >> (8 * (j & 3))) & 0xffu);
            const int32_t x = args.res_unsigned ? (int32_t)b : (int32_t)(int8_t)b;
            const int32_t v = ((q[j] * args.add_m_self + hs) >> args.add_s_self) + ((x * args.add_m_res + hr) >> args.add_s_res);
            q[j] = min(max(v, args.add_lo), args.add_hi);
          }
        }
        if (args.out_mode == IGEMM_OUT_NCHW) {
          if (row_valid) {
            const long long off0 = out_base + (long long)(n0 + cbase) * chan_stride;
            if (out8) {
              uint8_t* o = reinterpret_cast<uint8_t*>(args.out) + off0;
              if (ncols == CH && args.out_small) {
                // whole output below 2^31 elements: uniform base + 32-bit per-thread offsets
                uint8_t* const ob = reinterpret_cast<uint8_t*>(args.out);
                uint32_t off = (uint32_t)off0;
#pragma unroll
                for (int j = 0; j < CH; ++j, off += (uint32_t)chan_stride) ob[off] = (uint8_t)q[j];
              } else if (ncols == CH) {
#pragma unroll
                for (int j = 0; j < CH; ++j, o += chan_stride) *o = (uint8_t)q[j];
              } else {
#pragma unroll
                for (int j = 0; j < CH; ++j)
                  if (j < ncols) o[j * chan_stride] = (uint8_t)q[j];
              }
            } else if (e.out_dtype == B200Q_DT_I32) {
              int32_t* o = reinterpret_cast<int32_t*>(args.out) + off0;
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (j < ncols) o[j * chan_stride] = q[j];
            } else {
              uint16_t* o = reinterpret_cast<uint16_t*>(args.out) + off0;
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (j < ncols) o[j * chan_stride] = (uint16_t)q[j];
            }
          }
        } else if (row_valid || write_zero_row) {
          if (write_zero_row) {
#pragma unroll
            for (int j = 0; j < CH; ++j) q[j] = 0;
          }
          const long long off = out_base + n0 + cbase;
          if (out8) {
            uint8_t* o = reinterpret_cast<uint8_t*>(args.out) + off;
            if (ncols == CH && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
              uint32_t p[CH / 4];
              if (raw && e.out_dtype == B200Q_DT_U8) {
#pragma unroll
                for (int j = 0; j < CH / 4; ++j) p[j] = ptx::pack4_sat_u8(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
              } else if (raw) {
#pragma unroll
                for (int j = 0; j < CH / 4; ++j) p[j] = ptx::pack4_sat_s8(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < CH / 4; ++j)
                  p[j] = (uint32_t)(q[4 * j] & 0xff) | ((uint32_t)(q[4 * j + 1] & 0xff) << 8) |
                         ((uint32_t)(q[4 * j + 2] & 0xff) << 16) | ((uint32_t)(q[4 * j + 3] & 0xff) << 24);
              }
              reinterpret_cast<uint4*>(o)[0] = make_uint4(p[0], p[1], p[2], p[3]);
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (j < ncols) o[j] = (uint8_t)(raw ? min(max(q[j], sat_lo2), sat_hi) : q[j]);
            }
          } else if (e.out_dtype == B200Q_DT_I32) {
            int32_t* o = reinterpret_cast<int32_t*>(args.out) + off;
            if (ncols == CH && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < CH / 4; ++j)
                reinterpret_cast<int4*>(o)[j] = make_int4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (j < ncols) o[j] = q[j];
            }
          } else {
            uint16_t* o = reinterpret_cast<uint16_t*>(args.out) + off;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (j < ncols) o[j] = (uint16_t)q[j];
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  // a wait that ran out in one CTA of a pair ends the other CTA's waits too (they poll their own flag)
  if (PAIR && *abort_flag != 0) ptx::st_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32((const void*)abort_flag), cta_rank ^ 1u), (uint32_t)*abort_flag);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();  // neither CTA frees TMEM or exits while the other can still signal or read it
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TmemCols<BLOCK_N>::value);
    else ptx::tmem_dealloc(tmem_base, TmemCols<BLOCK_N>::value);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && args.status != nullptr) atomicCAS(args.status, 0, *abort_flag);
}
#undef floor_pre
#undef sat_lo2
#undef sat_hi
#undef pack_sat
#undef floor_needed

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D uint8 tensor [outer][inner] with row pitch `pitch` bytes, box {128 bytes, box_rows}, 128-byte swizzle.
int make_tmap_u8_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch,
                    uint32_t box_rows) {
  const uint64_t dims[2] = {inner, outer};
  const uint64_t strides[1] = {pitch};
  const uint32_t box[2] = {(uint32_t)BLOCK_K, box_rows};
  return make_tmap_u8(map, base, 2, dims, strides, box);
}

template <int BLOCK_N, int STAGES, int DIALECT, int RMODE, bool PAIR, int TAPW, bool PERROW = false, bool ADD = false>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const IGemmArgs& args, int workers, cudaStream_t stream) {
  using L = SmemLayout<BLOCK_N, STAGES, PAIR, TAPW>;
  auto kfn = igemm_i8_kernel<BLOCK_N, STAGES, DIALECT, RMODE, PAIR, TAPW, PERROW, ADD>;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(PAIR ? 2 * workers : workers);
  cfg.blockDim = dim3(L::NUM_THREADS);
  cfg.dynamicSmemBytes = L::DYN_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // after a kernel that releases its dependents early (the layout kernel of a convolution): this grid may become
  // resident and set itself up while that kernel drains; every role waits before its first global access
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = args.dependent_launch ? 2 : 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kfn, ta, tb, args));
  return B200Q_OK;
}

template <int BLOCK_N, int STAGES, bool PAIR, int TAPW = 1>
int launch_dialect(const CUtensorMap& ta, const CUtensorMap& tb, const IGemmArgs& a, int workers, cudaStream_t s) {
  const int d = a.epi.dialect, r = a.epi.round_mode;
  if (a.bf16) return launch_one<BLOCK_N, STAGES, KIND_BF16_TAG, -1, PAIR, TAPW>(ta, tb, a, workers, s);
  if (a.res != nullptr) {   // the fused residual Add is built for the dialect the BM168x lowering emits
    if (d == B200Q_RQ_MULTIPLIER_SHIFT && r == B200Q_ROUND_HALF_UP && !a.bf16)
      return launch_one<BLOCK_N, STAGES, B200Q_RQ_MULTIPLIER_SHIFT, B200Q_ROUND_HALF_UP, PAIR, TAPW, false, true>(ta, tb, a, workers, s);
    return set_error(B200Q_ERR_UNSUPPORTED, "igemm: the fused Add exists for MultiplierShift / half-up requantisation only");
  }
  if (d == B200Q_RQ_MULTIPLIER_SHIFT && r == B200Q_ROUND_HALF_UP)
    return launch_one<BLOCK_N, STAGES, B200Q_RQ_MULTIPLIER_SHIFT, B200Q_ROUND_HALF_UP, PAIR, TAPW>(ta, tb, a, workers, s);
  if (d == B200Q_RQ_QDM && r == B200Q_ROUND_HALF_AWAY_FROM_ZERO)
    return launch_one<BLOCK_N, STAGES, B200Q_RQ_QDM, B200Q_ROUND_HALF_AWAY_FROM_ZERO, PAIR, TAPW>(ta, tb, a, workers, s);
  return launch_one<BLOCK_N, STAGES, -1, -1, PAIR, TAPW>(ta, tb, a, workers, s);
}

// per-row parameters: built for the two dialects that have fast forms
template <int BLOCK_N, int STAGES, bool PAIR>
int launch_per_row(const CUtensorMap& ta, const CUtensorMap& tb, const IGemmArgs& a, int workers, cudaStream_t s) {
  const int d = a.epi.dialect, r = a.epi.round_mode;
  if (a.res != nullptr) {
    if (d == B200Q_RQ_MULTIPLIER_SHIFT && r == B200Q_ROUND_HALF_UP)
      return launch_one<BLOCK_N, STAGES, B200Q_RQ_MULTIPLIER_SHIFT, B200Q_ROUND_HALF_UP, PAIR, 1, true, true>(ta, tb, a, workers, s);
    return set_error(B200Q_ERR_UNSUPPORTED, "igemm: the fused Add exists for MultiplierShift / half-up requantisation only");
  }
  if (d == B200Q_RQ_MULTIPLIER_SHIFT && r == B200Q_ROUND_HALF_UP)
    return launch_one<BLOCK_N, STAGES, B200Q_RQ_MULTIPLIER_SHIFT, B200Q_ROUND_HALF_UP, PAIR, 1, true>(ta, tb, a, workers, s);
  if (d == B200Q_RQ_QDM && r == B200Q_ROUND_HALF_AWAY_FROM_ZERO)
    return launch_one<BLOCK_N, STAGES, B200Q_RQ_QDM, B200Q_ROUND_HALF_AWAY_FROM_ZERO, PAIR, 1, true>(ta, tb, a, workers, s);
  return set_error(B200Q_ERR_UNSUPPORTED, "igemm: per-row parameters exist for MultiplierShift/half-up and QDM/half-away only");
}

}  // namespace

// uint8 tensor map of `rank` dimensions (dims[0] innermost, strides_bytes[i] = byte pitch of dimension i+1), 128-byte
// swizzle, zero fill outside the tensor.  box[0] must be 128 (one swizzle span).
int make_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                 const uint32_t* box) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return set_error(B200Q_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return set_error(B200Q_ERR_INVALID, "TMA operand base %p is not 16-byte aligned", base);
  cuuint64_t d[5];
  cuuint64_t st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      st[i] = strides_bytes[i];
      if (st[i] & 15) return set_error(B200Q_ERR_INVALID, "TMA operand pitch %llu is not a multiple of 16 bytes", (unsigned long long)st[i]);
    }
  }
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), d, st, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200Q_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return B200Q_OK;
}

// B200Q_IGEMM_TAPFUSE=0 in the environment keeps 3-tap filter rows on one activation load per tap (for A/B timing).
// Test aid: launches wait for `extra` bytes more than their loads deliver, for at most `budget_ns` (0 = default).
static std::atomic<unsigned long long> g_wait_budget_ns{DEFAULT_WAIT_BUDGET_NS};
static std::atomic<int> g_expect_extra{0};
void igemm_set_wait_test(int extra_tx_bytes, long long budget_ns) {
  g_expect_extra.store(extra_tx_bytes < 0 ? 0 : extra_tx_bytes, std::memory_order_relaxed);
  g_wait_budget_ns.store(budget_ns > 0 ? (unsigned long long)budget_ns : DEFAULT_WAIT_BUDGET_NS, std::memory_order_relaxed);
}

static bool tapfuse_allowed() {
  static const bool on = [] {
    const char* v = getenv("B200Q_IGEMM_TAPFUSE");
    return !(v && v[0] == '0');
  }();
  return on;
}

// B200Q_IGEMM_PAIR=0 in the environment keeps every launch on single-CTA tiles (for A/B timing).
static bool pair_mode_allowed() {
  static const bool on = [] {
    const char* v = getenv("B200Q_IGEMM_PAIR");
    return !(v && v[0] == '0');
  }();
  return on;
}

int igemm_i8_tcgen05_supported(const IGemmProblem& p, const char** why) {
  const char* w = nullptr;
  if (p.k_per_tap % 16 != 0) w = "K (channels per filter tap) must be a multiple of 16 bytes";
  else if (p.taps_h * p.taps_w > 1 && p.k_per_tap % BLOCK_K != 0) w = "multi-tap convolution needs C % 128 == 0";
  else if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15)) w = "unaligned operand";
  else if (p.a_pitch % 16 != 0 || p.b_pitch % 16 != 0) w = "operand row pitch must be a multiple of 16 bytes";
  else if (p.rows <= 0 || p.n <= 0) w = "empty problem";
  if (why) *why = w;
  return w == nullptr;
}

// Launch the tcgen05 implicit GEMM.  Asynchronous on `stream`; `status` (device int, may be null) receives a
// non-zero code if a bounded wait inside the kernel ran out.
int igemm_i8_tcgen05_launch(const IGemmProblem& p, const Epilogue& epi, int* status, cudaStream_t stream) {
  const char* why = nullptr;
  if (!igemm_i8_tcgen05_supported(p, &why)) return set_error(B200Q_ERR_UNSUPPORTED, "tcgen05 igemm: %s", why);
  const int block_n = p.n > 128 ? 256 : (p.n > 64 ? 128 : 64);
  const int kb_per_tap = (p.k_per_tap + BLOCK_K - 1) / BLOCK_K;

  IGemmArgs a{};
  a.rows = p.rows;
  a.n = p.n;
  a.kb_per_tap = kb_per_tap;
  a.taps_w = p.taps_w;
  a.tap_step_w = p.tap_step_w > 0 ? p.tap_step_w : 1;
  a.num_kb = kb_per_tap * p.taps_h * p.taps_w;
  a.tap_org_h = p.pad_top;
  a.tap_org_w = p.pad_left;
  a.row_pitch = p.row_pitch > 0 ? p.row_pitch : 1;
  a.out_mode = p.out_mode;
  a.img_rows = p.img_rows > 0 ? p.img_rows : 1;
  a.border_h = p.border_h;
  a.border_w = p.border_w;
  a.out_h = p.out_h;
  a.out_w = p.out_w;
  a.ldc = p.ldc;
  a.out = p.out;
  a.epi = epi;
  a.status = status;
  a.res = static_cast<const uint8_t*>(p.res);
  if (p.res != nullptr) {
    const bool out8 = epi.out_dtype == B200Q_DT_I8 || epi.out_dtype == B200Q_DT_U8;
    auto m_ok = [](int m) { return m > -(1 << 23) && m < (1 << 23); };
    auto s_ok = [](int sft) { return sft >= 1 && sft <= 31; };
    if (!out8 || p.kind != IGEMM_KIND_I8 || !m_ok(p.add_m_self) || !m_ok(p.add_m_res) || !s_ok(p.add_s_self) || !s_ok(p.add_s_res) ||
        p.out_mode == IGEMM_OUT_NHWC_BORDERED)
      return set_error(B200Q_ERR_UNSUPPORTED, "tcgen05 igemm: fused Add needs 8-bit tensors, |multiplier| < 2^23, shifts in [1,31]");
    a.res_unsigned = p.res_unsigned;
    a.add_m_self = p.add_m_self;
    a.add_s_self = p.add_s_self;
    a.add_m_res = p.add_m_res;
    a.add_s_res = p.add_s_res;
    a.add_lo = p.add_lo;
    a.add_hi = p.add_hi;
  }
  a.wait_budget_ns = g_wait_budget_ns.load(std::memory_order_relaxed);
  a.expect_extra = g_expect_extra.load(std::memory_order_relaxed);
  a.bf16 = p.kind == IGEMM_KIND_BF16 || p.kind == IGEMM_KIND_F16;
  a.f16 = p.kind == IGEMM_KIND_F16;
  // |accumulator| < 2^29 for every 8-bit operand pair: lets the epilogue fold the bias into one 64-bit constant
  // largest |a * b| of one product: 255 * 255 for two unsigned operands, 255 * 128 mixed, 128 * 128 for two signed ones
  const long long max_prod = (p.a_unsigned && p.b_unsigned) ? 65025ll : ((p.a_unsigned || p.b_unsigned) ? 32640ll : 16384ll);
  a.acc_small = ((long long)a.num_kb * BLOCK_K * max_prod) < (1ll << 29);
  {
    int lo, hi;
    switch (epi.out_dtype) {
      case B200Q_DT_I8: lo = -128; hi = 127; break;
      case B200Q_DT_U8: lo = 0; hi = 255; break;
      case B200Q_DT_I16: lo = -32768; hi = 32767; break;
      case B200Q_DT_U16: lo = 0; hi = 65535; break;
      default: lo = -2147483647 - 1; hi = 2147483647; break;
    }
    const int floor_post = epi.relu == B200Q_RELU_AFTER_REQUANT ? epi.out_zp : (-2147483647 - 1);
    const bool out8 = epi.out_dtype == B200Q_DT_I8 || epi.out_dtype == B200Q_DT_U8;
    a.floor_pre = epi.relu == B200Q_RELU_BEFORE_REQUANT ? 0 : (-2147483647 - 1);
    a.sat_hi = hi;
    a.sat_lo2 = lo > floor_post ? lo : floor_post;
    a.pack_sat = out8 && p.out_mode != IGEMM_OUT_NCHW;
    a.floor_needed = a.sat_lo2 > lo;
  }
  a.dependent_launch = p.dependent_launch;
  a.acc_bound = a.acc_small ? (int)((long long)a.num_kb * BLOCK_K * max_prod) : (1 << 29);
  a.bias_f32 = p.bias_f32;
  {
    const long long out_elems = p.out_mode == IGEMM_OUT_NCHW
                                    ? (((long long)p.rows + a.img_rows - 1) / a.img_rows) * p.n * p.out_h * p.out_w
                                    : (long long)p.rows * p.ldc;  // (an upper bound for IGEMM_OUT_NHWC)
    a.out_small = out_elems < (1ll << 31);
  }
  // CTA pairs (256-row tiles, cta_group::2) once there is more than one wave of 128-row tiles to share out
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long tiles128 = (long long)((p.rows + BLOCK_M - 1) / BLOCK_M) * ((p.n + block_n - 1) / block_n);
  const bool pair = block_n == 256 && pair_mode_allowed() && tiles128 >= 2ll * sms && p.rows > BLOCK_M;
  // three taps per filter row, one pixel apart, no ragged K block: the taps of a row share one activation block
  const bool tapfuse = pair && tapfuse_allowed() && p.taps_w == 3 && a.tap_step_w == 1 && p.k_per_tap % BLOCK_K == 0 && !a.bf16;
  const int tile_m = pair ? 2 * BLOCK_M : BLOCK_M;
  a.idesc = a.bf16 ? ptx::make_idesc(1u, a.f16 ? 0u : 1u, a.f16 ? 0u : 1u, tile_m, (uint32_t)block_n)  // f32 accumulate, bf16 x bf16 or f16 x f16
                   : ptx::make_idesc(2u, p.a_unsigned ? 0u : 1u, p.b_unsigned ? 0u : 1u, tile_m, (uint32_t)block_n);
  a.num_m_tiles = (p.rows + tile_m - 1) / tile_m;
  a.num_n_tiles = (p.n + block_n - 1) / block_n;
  {
    // band height of the tile walk: a wave of tiles (one per worker) whose A rows and B rows cost about the same would
    // be sqrt(workers * block_n / tile_m) row tiles high; twice that measured best on the 8192^3 GEMM (bands of 8 / 12 /
    // 16 / 24 / 32 row tiles: 3092 / 3127 / 3172 / 3127 / 2993 TOPS, row-major walk 2952).  B200Q_IGEMM_BAND=<n>
    // overrides (1 = the row-major walk), for A/B timing.
    const int workers_est = pair ? sms / 2 : sms;
    int band = (int)(2.0 * sqrt((double)workers_est * block_n / tile_m) + 0.5);
    static const int band_env = [] {
      const char* v = getenv("B200Q_IGEMM_BAND");
      return v ? atoi(v) : 0;
    }();
    if (band_env > 0) band = band_env;
    a.band_m = a.num_n_tiles > 1 ? (band < a.num_m_tiles ? band : a.num_m_tiles) : 1;
  }

  CUtensorMap ta, tb;
  // (a_pitch < k_per_tap: overlapping rows, each spanning several consecutive pixels; the caller keeps
  // k_per_tap - a_pitch readable bytes behind the last row)
  int rc = make_tmap_u8_2d(&ta, p.a, (uint64_t)p.k_per_tap, (uint64_t)p.rows, (uint64_t)p.a_pitch,
                           tapfuse ? BLOCK_M + 2 : BLOCK_M);
  if (rc) return rc;
  // B: [n][taps * k_per_tap]; with several taps k_per_tap is a multiple of BLOCK_K so blocks never straddle taps
  rc = make_tmap_u8_2d(&tb, p.b, (uint64_t)p.k_per_tap * p.taps_h * p.taps_w, (uint64_t)p.n, (uint64_t)p.b_pitch,
                       (uint32_t)(pair ? block_n / 2 : block_n));
  if (rc) return rc;

  const int tiles = a.num_m_tiles * a.num_n_tiles;
  const int slots = pair ? sms / 2 : sms;
  const int workers = tiles < slots ? tiles : slots;
  if (p.per_row_params) {
    if (a.bf16 || block_n != 256) return set_error(B200Q_ERR_UNSUPPORTED, "igemm: per-row parameters need the 256-column tile");
    return pair ? launch_per_row<256, 6, true>(ta, tb, a, workers, stream) : launch_per_row<256, 4, false>(ta, tb, a, workers, stream);
  }
  if (tapfuse) return launch_dialect<256, 3, true, 3>(ta, tb, a, workers, stream);
  if (pair) return launch_dialect<256, 6, true>(ta, tb, a, workers, stream);
  switch (block_n) {
    case 256: return launch_dialect<256, 4, false>(ta, tb, a, workers, stream);
    case 128: return launch_dialect<128, 6, false>(ta, tb, a, workers, stream);
    default: return launch_dialect<64, 8, false>(ta, tb, a, workers, stream);
  }
}

}  // namespace b200q
