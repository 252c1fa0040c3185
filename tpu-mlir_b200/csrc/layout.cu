// Data-movement kernels around the tensor-core path: layout changes between the interpreter's NCHW
// tensors and the zero-bordered NHWC image the implicit GEMM reads, weight repacking (once per op),
// and the float <-> native-integer conversions of the operator face (the interpreter keeps every tensor,
// integer ones included, as float: bindings/pymlir/host/ModuleInterpreter.cpp:396-492).
#include <cstdlib>
#include "internal.h"
#include "layout.h"

namespace b200q {
namespace {

template <typename T>
__device__ __forceinline__ uint8_t to_byte(T v);
template <>
__device__ __forceinline__ uint8_t to_byte<uint8_t>(uint8_t v) { return v; }
template <>
__device__ __forceinline__ uint8_t to_byte<float>(float v) { return (uint8_t)(int)v; }  // integral by contract

// x[N][C][H][W] -> y[N][H+2bh][W+2bw][C] interior (the border is zeroed once when the buffer is created).
// Tile of 32 channels x 32 pixels of one image row through shared memory: reads run along W, writes along C.
template <typename T>
__global__ void nchw_to_bordered_nhwc_kernel(const T* __restrict__ x, uint8_t* __restrict__ y, int C, int H, int W,
                                             int bh, int bw) {
  __shared__ uint8_t tile[32][33];
  const int Wp = W + 2 * bw, Hp = H + 2 * bh;
  const int w0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int nh = blockIdx.z;
  const int n = nh / H, h = nh - n * H;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, w = w0 + tx;
    tile[i][tx] = (c < C && w < W) ? to_byte<T>(x[(((long long)n * C + c) * H + h) * W + w]) : (uint8_t)0;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int w = w0 + i, c = c0 + tx;
    if (w < W && c < C) y[(((long long)n * Hp + (h + bh)) * Wp + (w + bw)) * C + c] = tile[tx][i];
  }
}


// Fast path of the same transform for H*W % 4 == 0 and C % 4 == 0: a block moves 128 channels x 128 pixels.
// Reads are 128-byte (512-byte for float input) coalesced runs along W, a 4x4 byte transpose happens in
// registers (prmt), the tile goes through XOR-swizzled shared memory, and writes are 128-byte runs along C.
template <typename T>
struct Pix4;
template <>
struct Pix4<uint8_t> {
  static __device__ __forceinline__ uint32_t load(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
};
template <>
struct Pix4<float> {
  static __device__ __forceinline__ uint32_t load(const float* p) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    return (uint32_t)((int)v.x & 0xff) | ((uint32_t)((int)v.y & 0xff) << 8) | ((uint32_t)((int)v.z & 0xff) << 16) |
           ((uint32_t)((int)v.w & 0xff) << 24);
  }
};

template <typename T>
__global__ void __launch_bounds__(256)
nchw_to_bordered_nhwc_fast_kernel(const T* __restrict__ x, uint8_t* __restrict__ y, int C, int H, int W, int bh, int bw) {
  __shared__ uint32_t tile[128][32];  // [pixel][4-channel word], word column XORed with (pixel >> 2) & 31
  const int HW = H * W, Wp = W + 2 * bw, Hp = H + 2 * bh;
  const int p0 = blockIdx.x * 128, c0 = blockIdx.y * 128, n = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pix = p0 + 4 * lane;  // this lane's 4 pixels
  const T* xn = x + (long long)n * C * HW;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int cg = warp * 4 + g;  // channel group of 4 (word column)
    const int c = c0 + 4 * cg;
    uint32_t a = 0, b = 0, cc = 0, d = 0;
    if (pix < HW && c < C) {  // C % 4 == 0: a group is entirely inside or outside
      a = Pix4<T>::load(xn + (long long)(c + 0) * HW + pix);
      b = Pix4<T>::load(xn + (long long)(c + 1) * HW + pix);
      cc = Pix4<T>::load(xn + (long long)(c + 2) * HW + pix);
      d = Pix4<T>::load(xn + (long long)(c + 3) * HW + pix);
    }
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(cc, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(cc, d, 0x7362);
    const int col = cg ^ lane;  // (pixel >> 2) & 31 == lane for all four pixels of this lane
    tile[4 * lane + 0][col] = __byte_perm(t0, t1, 0x5410);
    tile[4 * lane + 1][col] = __byte_perm(t0, t1, 0x7632);
    tile[4 * lane + 2][col] = __byte_perm(t2, t3, 0x5410);
    tile[4 * lane + 3][col] = __byte_perm(t2, t3, 0x7632);
  }
  __syncthreads();
  uint8_t* yn = y + (long long)n * Hp * Wp * C;
  for (int r = warp; r < 128; r += 8) {
    const int p = p0 + r;
    if (p >= HW) break;
    const int h = p / W, w = p - h * W;
    const int cg = lane ^ ((r >> 2) & 31);
    const int c = c0 + 4 * cg;
    if (c < C)
      *reinterpret_cast<uint32_t*>(yn + ((long long)(h + bh) * Wp + (w + bw)) * C + c) = tile[r][lane];
  }
}

// Wider variant for C % 16 == 0 and H*W % 16 == 0: a thread reads 4 channels x 16 pixels as 16-byte runs, transposes
// four 4x4 byte blocks in registers and parks them in the same XOR-swizzled tile; then every thread writes 16
// channels of one pixel with one 16-byte store (4 pixels x 128 channels per warp instruction).
template <typename T>
struct Pix16;
template <>
struct Pix16<uint8_t> {
  static __device__ __forceinline__ uint4 load(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
};
template <>
struct Pix16<float> {
  static __device__ __forceinline__ uint4 load(const float* p) {
    return make_uint4(Pix4<float>::load(p), Pix4<float>::load(p + 4), Pix4<float>::load(p + 8), Pix4<float>::load(p + 12));
  }
};

// TILES pixel tiles of 128 per block.  Two tiles (all loads issued before the first transposition, 832 blocks for a
// 32 x 256 x 56 x 56 image, all resident at once) were measured against one tile (1600 blocks): 19.0 us against 15.1 us
// inside the convolution step, so one tile is what runs; B200Q_LAYOUT_TILES=2 selects the other for A/B timing.
// (Half-size blocks, 64 pixels and 128 threads, measured the same as one tile: 15.0-15.1 us.)
template <typename T, int TILES>
__global__ void __launch_bounds__(256)
nchw_to_bordered_nhwc_wide_kernel(const T* __restrict__ x, uint8_t* __restrict__ y, int C, int H, int W, int bh, int bw) {
  __shared__ uint32_t tile[TILES][128][32];  // [pixel][4-channel word], word column XORed with (pixel >> 2) & 31
  // The convolution kernel that follows may become resident while this grid drains (it waits for this grid's
  // completion before it reads the image).  (Launching this grid itself as a programmatic dependent of the previous
  // convolution was measured and dropped: 54.6-55.1 us per step against 53.2 us.)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int HW = H * W, Wp = W + 2 * bw, Hp = H + 2 * bh;
  const int p0 = blockIdx.x * (128 * TILES), c0 = blockIdx.y * 128, n = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const int cg = threadIdx.x >> 3;  // channel group of 4 (word column), 0..31
    const int pc = threadIdx.x & 7;   // 16-pixel chunk of the tile
    const int c = c0 + 4 * cg;
    uint4 ch[TILES][4];
#pragma unroll
    for (int u = 0; u < TILES; ++u) {
      const int pix = p0 + 128 * u + 16 * pc;
#pragma unroll
      for (int i = 0; i < 4; ++i) ch[u][i] = make_uint4(0, 0, 0, 0);
      if (pix < HW && c < C) {  // H*W % 16 == 0 and C % 4 == 0: a chunk / group is entirely inside or outside
        const T* src = x + ((long long)n * C + c) * HW + pix;
#pragma unroll
        for (int i = 0; i < 4; ++i) ch[u][i] = Pix16<T>::load(src + (long long)i * HW);
      }
    }
#pragma unroll
    for (int u = 0; u < TILES; ++u) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {  // pixels 4*q4 .. 4*q4+3 of the chunk
        const uint32_t a = (&ch[u][0].x)[q4], b = (&ch[u][1].x)[q4], cc = (&ch[u][2].x)[q4], d = (&ch[u][3].x)[q4];
        const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(cc, d, 0x5140);
        const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(cc, d, 0x7362);
        const int row = 16 * pc + 4 * q4;
        const int col = cg ^ ((row >> 2) & 31);
        tile[u][row + 0][col] = __byte_perm(t0, t1, 0x5410);
        tile[u][row + 1][col] = __byte_perm(t0, t1, 0x7632);
        tile[u][row + 2][col] = __byte_perm(t2, t3, 0x5410);
        tile[u][row + 3][col] = __byte_perm(t2, t3, 0x7632);
      }
    }
  }
  __syncthreads();
  uint8_t* yn = y + (long long)n * Hp * Wp * C;
  const int k = lane & 7;  // 16-channel chunk of the pixel
  const int c = c0 + 16 * k;
#pragma unroll
  for (int u = 0; u < TILES; ++u) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // the four pixel rows a warp reads at once lie in four different swizzle groups: no bank conflicts
      const int r = warp * 16 + (lane >> 3) * 4 + i;
      const int p = p0 + 128 * u + r;
      if (p < HW && c < C) {
        const int sw = (r >> 2) & 31;
        const uint4 v = make_uint4(tile[u][r][(4 * k + 0) ^ sw], tile[u][r][(4 * k + 1) ^ sw], tile[u][r][(4 * k + 2) ^ sw],
                                   tile[u][r][(4 * k + 3) ^ sw]);
        const int h = p / W, w = p - h * W;
        *reinterpret_cast<uint4*>(yn + ((long long)(h + bh) * Wp + (w + bw)) * C + c) = v;
      }
    }
  }
}

// Small images with any H*W (7x7 and the like), C % 64 == 0: a block takes 64 channels of one image, which are one
// contiguous run of 64*H*W source elements, parks them as bytes in shared memory with 4-element accesses, and writes
// every pixel's 64 channels as 16 four-byte words (64 contiguous bytes per pixel).
template <typename T>
__global__ void __launch_bounds__(256)
nchw_to_bordered_nhwc_small_kernel(const T* __restrict__ x, uint8_t* __restrict__ y, int C, int H, int W, int bh, int bw) {
  extern __shared__ __align__(16) uint8_t stile[];  // [64][H*W]
  const int HW = H * W, Wp = W + 2 * bw, Hp = H + 2 * bh;
  const int c0 = blockIdx.x * 64, n = blockIdx.y;
  const T* src = x + ((long long)n * C + c0) * HW;
  const int words = 16 * HW;  // 64*HW bytes
  for (int i = threadIdx.x; i < words; i += 256)
    reinterpret_cast<uint32_t*>(stile)[i] = Pix4<T>::load(src + 4 * i);
  __syncthreads();
  uint8_t* yn = y + (long long)n * Hp * Wp * C + c0;
  for (int i = threadIdx.x; i < words; i += 256) {
    const int p = i >> 4, wq = i & 15;
    const uint8_t* t = stile + (4 * wq) * HW + p;
    const uint32_t v = (uint32_t)t[0] | ((uint32_t)t[HW] << 8) | ((uint32_t)t[2 * HW] << 16) | ((uint32_t)t[3 * HW] << 24);
    const int h = p / W, w = p - h * W;
    *reinterpret_cast<uint32_t*>(yn + ((long long)(h + bh) * Wp + (w + bw)) * C + 4 * wq) = v;
  }
}

// w[OC][IC][KH][KW] -> wr[OC][KH*KW][IC]  (K-major rows for the implicit GEMM: k = tap * IC + ic)
template <typename T>
__global__ void repack_weight_kernel(const T* __restrict__ w, uint8_t* __restrict__ wr, int OC, int IC, int KHW) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)OC * IC * KHW;
  if (idx >= total) return;
  const int ic = (int)(idx % IC);
  const int tap = (int)((idx / IC) % KHW);
  const int oc = (int)(idx / ((long long)IC * KHW));
  wr[idx] = to_byte<T>(w[((long long)oc * IC + ic) * KHW + tap]);
}

// 64-channel filters with horizontally adjacent taps paired into one 128-byte K block:
// w[OC][64][KH][KW] -> wr[OC][KH][ceil(KW/2)][2][64], a missing second tap (odd KW) is zero.
template <typename T>
__global__ void repack_weight_pairs_kernel(const T* __restrict__ w, uint8_t* __restrict__ wr, int OC, int KH, int KW) {
  const int KW2 = (KW + 1) / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)OC * KH * KW2 * 128;
  if (idx >= total) return;
  const int ic = (int)(idx % 64);
  const int sub = (int)((idx / 64) % 2);
  const int fx2 = (int)((idx / 128) % KW2);
  const int fy = (int)((idx / (128LL * KW2)) % KH);
  const int oc = (int)(idx / (128LL * KW2 * KH));
  const int fx = 2 * fx2 + sub;
  wr[idx] = fx < KW ? to_byte<T>(w[(((long long)oc * 64 + ic) * KH + fy) * KW + fx]) : (uint8_t)0;
}

// filters for the few-channel im2col: w[OC][C][KH][KW] -> wr[OC][kpad], k = (fy*C + c)*8 + fx, zero elsewhere
template <typename T>
__global__ void repack_weight_fy_c_fx8_kernel(const T* __restrict__ w, uint8_t* __restrict__ wr, int OC, int C, int KH, int KW,
                                              int kpad) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)OC * kpad) return;
  const int k = (int)(idx % kpad), oc = (int)(idx / kpad);
  const int fx = k & 7, seg = k >> 3;
  uint8_t v = 0;
  if (seg < KH * C && fx < KW) {
    const int fy = seg / C, c = seg - fy * C;
    v = to_byte<T>(w[(((long long)oc * C + c) * KH + fy) * KW + fx]);
  }
  wr[idx] = v;
}

// [rows][cols] bytes -> [cols][rows] bytes
template <typename T>
__global__ void transpose_to_u8_kernel(const T* __restrict__ src, uint8_t* __restrict__ dst, int rows, int cols) {
  __shared__ uint8_t tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    tile[i][tx] = (r < rows && c < cols) ? to_byte<T>(src[(long long)r * cols + c]) : (uint8_t)0;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + tx;
    if (c < cols && r < rows) dst[(long long)c * rows + r] = tile[tx][i];
  }
}

__global__ void f32_to_q8_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = (uint8_t)(int)x[i];
}
__global__ void f32_to_i32_kernel(const float* __restrict__ x, int32_t* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = (int32_t)x[i];
}
__global__ void q_to_f32_kernel(const void* __restrict__ x, int dt, float* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  switch (dt) {
    case B200Q_DT_I8: y[i] = (float)reinterpret_cast<const int8_t*>(x)[i]; break;
    case B200Q_DT_U8: y[i] = (float)reinterpret_cast<const uint8_t*>(x)[i]; break;
    case B200Q_DT_I16: y[i] = (float)reinterpret_cast<const int16_t*>(x)[i]; break;
    case B200Q_DT_U16: y[i] = (float)reinterpret_cast<const uint16_t*>(x)[i]; break;
    default: y[i] = (float)reinterpret_cast<const int32_t*>(x)[i]; break;
  }
}

inline unsigned blocks_for(long long n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

int nchw_to_bordered_nhwc(const void* x, int x_is_f32, void* y, int N, int C, int H, int W, int bh, int bw,
                          cudaStream_t s) {
  const long long HW = (long long)H * W;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % (x_is_f32 ? 16 : 4) == 0) && (reinterpret_cast<uintptr_t>(y) % 4 == 0);
  if (HW % 16 == 0 && C % 16 == 0 && N <= 65535 && ceil_div(C, 128) <= 65535 &&
      reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
    const long long blocks1 = (long long)ceil_div(HW, 128) * ceil_div(C, 128) * N;
    static const int force_tiles = [] {
      const char* v = getenv("B200Q_LAYOUT_TILES");   // 1 or 2: A/B timing
      return v ? atoi(v) : 0;
    }();
    const bool two = force_tiles == 2 && blocks1 >= 1024 && !x_is_f32;
    if (two) {
      dim3 grid(ceil_div(HW, 256), ceil_div(C, 128), N);
      nchw_to_bordered_nhwc_wide_kernel<uint8_t, 2><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, C, H, W, bh, bw);
    } else {
      dim3 grid(ceil_div(HW, 128), ceil_div(C, 128), N);
      if (x_is_f32)
        nchw_to_bordered_nhwc_wide_kernel<float, 1><<<grid, 256, 0, s>>>((const float*)x, (uint8_t*)y, C, H, W, bh, bw);
      else
        nchw_to_bordered_nhwc_wide_kernel<uint8_t, 1><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, C, H, W, bh, bw);
    }
    CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
  }
  if (HW % 16 != 0 && C % 64 == 0 && HW * 64 <= 48 * 1024 && N <= 65535 && aligned) {
    // (64 channels of one image start 64 elements-aligned: every 4-element load above is aligned)
    dim3 grid(C / 64, N);
    const size_t smem = (size_t)HW * 64;
    if (x_is_f32)
      nchw_to_bordered_nhwc_small_kernel<float><<<grid, 256, smem, s>>>((const float*)x, (uint8_t*)y, C, H, W, bh, bw);
    else
      nchw_to_bordered_nhwc_small_kernel<uint8_t><<<grid, 256, smem, s>>>((const uint8_t*)x, (uint8_t*)y, C, H, W, bh, bw);
    CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
  }
  if (HW % 4 == 0 && C % 4 == 0 && aligned && N <= 65535 && ceil_div(C, 128) <= 65535) {
    dim3 grid(ceil_div(HW, 128), ceil_div(C, 128), N);
    if (x_is_f32)
      nchw_to_bordered_nhwc_fast_kernel<float><<<grid, 256, 0, s>>>((const float*)x, (uint8_t*)y, C, H, W, bh, bw);
    else
      nchw_to_bordered_nhwc_fast_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, C, H, W, bh, bw);
    CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
  }
  if ((long long)N * H > 65535LL * 32767) return set_error(B200Q_ERR_UNSUPPORTED, "layout: N*H too large");
  dim3 grid(ceil_div(W, 32), ceil_div(C, 32), N * H), block(32, 8);
  if (grid.y > 65535 || grid.z > 65535) {
    // fold: z is limited to 65535; large batches are split
    const int per = 65535 / H > 0 ? 65535 / H : 1;
    for (int n0 = 0; n0 < N; n0 += per) {
      const int nn = (N - n0) < per ? (N - n0) : per;
      const long long xin = (long long)n0 * C * H * W, yout = (long long)n0 * (H + 2 * bh) * (W + 2 * bw) * C;
      B200Q_TRY(nchw_to_bordered_nhwc(x_is_f32 ? (const void*)((const float*)x + xin) : (const void*)((const uint8_t*)x + xin),
                                      x_is_f32, (uint8_t*)y + yout, nn, C, H, W, bh, bw, s));
    }
    return B200Q_OK;
  }
  if (x_is_f32)
    nchw_to_bordered_nhwc_kernel<float><<<grid, block, 0, s>>>((const float*)x, (uint8_t*)y, C, H, W, bh, bw);
  else
    nchw_to_bordered_nhwc_kernel<uint8_t><<<grid, block, 0, s>>>((const uint8_t*)x, (uint8_t*)y, C, H, W, bh, bw);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int repack_weight_oihw(const void* w, int w_is_f32, void* wr, int OC, int IC, int KH, int KW, cudaStream_t s) {
  const long long total = (long long)OC * IC * KH * KW;
  if (total == 0) return B200Q_OK;
  if (w_is_f32)
    repack_weight_kernel<float><<<blocks_for(total, 256), 256, 0, s>>>((const float*)w, (uint8_t*)wr, OC, IC, KH * KW);
  else
    repack_weight_kernel<uint8_t><<<blocks_for(total, 256), 256, 0, s>>>((const uint8_t*)w, (uint8_t*)wr, OC, IC, KH * KW);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int repack_weight_pairs64(const void* w, int w_is_f32, void* wr, int OC, int KH, int KW, cudaStream_t s) {
  const long long total = (long long)OC * KH * ((KW + 1) / 2) * 128;
  if (total == 0) return B200Q_OK;
  if (w_is_f32)
    repack_weight_pairs_kernel<float><<<blocks_for(total, 256), 256, 0, s>>>((const float*)w, (uint8_t*)wr, OC, KH, KW);
  else
    repack_weight_pairs_kernel<uint8_t><<<blocks_for(total, 256), 256, 0, s>>>((const uint8_t*)w, (uint8_t*)wr, OC, KH, KW);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int repack_weight_fy_c_fx8(const void* w, int w_is_f32, void* wr, int OC, int C, int KH, int KW, int kpad, cudaStream_t s) {
  const long long total = (long long)OC * kpad;
  if (total == 0) return B200Q_OK;
  if (w_is_f32)
    repack_weight_fy_c_fx8_kernel<float><<<blocks_for(total, 256), 256, 0, s>>>((const float*)w, (uint8_t*)wr, OC, C, KH, KW, kpad);
  else
    repack_weight_fy_c_fx8_kernel<uint8_t><<<blocks_for(total, 256), 256, 0, s>>>((const uint8_t*)w, (uint8_t*)wr, OC, C, KH, KW, kpad);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int transpose_to_u8(const void* src, int src_is_f32, void* dst, int rows, int cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return B200Q_OK;
  dim3 grid(ceil_div(cols, 32), ceil_div(rows, 32)), block(32, 8);
  if (grid.y > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "transpose: too many rows");
  if (src_is_f32) transpose_to_u8_kernel<float><<<grid, block, 0, s>>>((const float*)src, (uint8_t*)dst, rows, cols);
  else transpose_to_u8_kernel<uint8_t><<<grid, block, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, rows, cols);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// dst[c][r] = src[r][c] for float matrices (the output_transpose of tpu.MatMul, lib/Support/Dnnl/MatMul.cpp:229-238)
__global__ void transpose_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[(size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}

int transpose_f32(const float* src, float* dst, int rows, int cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return B200Q_OK;
  dim3 grid(ceil_div(cols, 32), ceil_div(rows, 32)), block(32, 8);
  if (grid.y > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "transpose: too many rows");
  transpose_f32_kernel<<<grid, block, 0, s>>>(src, dst, rows, cols);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int f32_to_q8(const float* x, void* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  f32_to_q8_kernel<<<blocks_for(n, 256), 256, 0, s>>>(x, (uint8_t*)y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}
int f32_to_i32(const float* x, int32_t* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  f32_to_i32_kernel<<<blocks_for(n, 256), 256, 0, s>>>(x, y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}
int q_to_f32(const void* x, int dt, float* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  q_to_f32_kernel<<<blocks_for(n, 256), 256, 0, s>>>(x, dt, y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
