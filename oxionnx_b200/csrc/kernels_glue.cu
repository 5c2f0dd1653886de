// Memory-bound glue kernels of the oxb200 path (sm_100a).  All of them stream their operands
// once through HBM with vectorised accesses where the layout allows; none of them uses a
// fused multiply-add (this file is compiled with --fmad=false) because the reference rounds
// every f32 operation separately and the quantisers sit right at rounding boundaries.
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.hpp"

namespace oxb {
namespace k {

namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t work, int per_block = kThreads) {
  int64_t b = (work + per_block - 1) / per_block;
  // Enough blocks to fill 148 SMs several times over, capped so the grid-stride loops stay
  // in a sane range for very large tensors.
  const int64_t cap = 148 * 64;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

__device__ __forceinline__ float load_as_f32(const void* p, DT dt, int64_t i) {
  switch (dt) {
    case DT::F32: return ((const float*)p)[i];
    case DT::U8: return (float)((const uint8_t*)p)[i];
    case DT::I8: return (float)((const int8_t*)p)[i];
    case DT::I32: return __int2float_rn(((const int32_t*)p)[i]);
    case DT::I16: return (float)((const int16_t*)p)[i];
  }
  return 0.f;
}

// Stores an f32 lane that holds an integer value (or a float for F32 storage).
__device__ __forceinline__ void store_from_f32(void* p, DT dt, int64_t i, float v) {
  switch (dt) {
    case DT::F32: ((float*)p)[i] = v; break;
    case DT::U8: ((uint8_t*)p)[i] = (uint8_t)__float2int_rn(fminf(fmaxf(v, 0.f), 255.f)); break;
    case DT::I8: ((int8_t*)p)[i] = (int8_t)__float2int_rn(fminf(fmaxf(v, -128.f), 127.f)); break;
    case DT::I32: ((int32_t*)p)[i] = __float2int_rn(v); break;
    case DT::I16: ((int16_t*)p)[i] = (int16_t)__float2int_rn(fminf(fmaxf(v, -32768.f), 32767.f)); break;
  }
}

struct Coord {
  int64_t n, c, h, w;
};

__device__ __forceinline__ Coord decode(int64_t o, Layout L, const Dims4& d) {
  Coord q;
  if (L == Layout::NHWC) {
    q.c = o % d.C;
    o /= d.C;
    q.w = o % d.W;
    o /= d.W;
    q.h = o % d.H;
    q.n = o / d.H;
  } else {
    q.w = o % d.W;
    o /= d.W;
    q.h = o % d.H;
    o /= d.H;
    q.c = o % d.C;
    q.n = o / d.C;
  }
  return q;
}

__device__ __forceinline__ int64_t encode(const Coord& q, Layout L, const Dims4& d) {
  if (L == Layout::NHWC) return ((q.n * d.H + q.h) * d.W + q.w) * d.C + q.c;
  return ((q.n * d.C + q.c) * d.H + q.h) * d.W + q.w;
}

// Offset of the broadcast source element for output coordinate q.
__device__ __forceinline__ int64_t encode_bcast(const Coord& q, Layout L, const Dims4& d) {
  Coord r;
  r.n = d.N == 1 ? 0 : q.n;
  r.c = d.C == 1 ? 0 : q.c;
  r.h = d.H == 1 ? 0 : q.h;
  r.w = d.W == 1 ? 0 : q.w;
  return encode(r, L, d);
}

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// ---------------------------------------------------------------------------------------
__global__ void convert_kernel(const void* src, DT sdt, Layout sl, void* dst, DT ddt, Layout dl, Dims4 d, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t si = o;
    if (sl != dl) si = encode(decode(o, dl, d), sl, d);
    float v = load_as_f32(src, sdt, si);
    if (sdt == DT::I32 && ddt == DT::I32) ((int32_t*)dst)[o] = ((const int32_t*)src)[si];
    else store_from_f32(dst, ddt, o, v);
  }
}

// NCHW -> NHWC (or back) through a shared-memory tile so both sides are coalesced.
// View: [outer, A, B] -> [outer, B, A]; 32x32 tiles.
template <typename TS, typename TD>
__global__ void transpose_tiles(const TS* __restrict__ src, TD* __restrict__ dst, int64_t A, int64_t B) {
  __shared__ float tile[32][33];
  int64_t outer = blockIdx.z;
  int64_t a0 = (int64_t)blockIdx.y * 32, b0 = (int64_t)blockIdx.x * 32;
  const TS* s = src + outer * A * B;
  TD* dptr = dst + outer * A * B;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int64_t a = a0 + i, b = b0 + threadIdx.x;
    if (a < A && b < B) tile[i][threadIdx.x] = (float)s[a * B + b];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int64_t b = b0 + i, a = a0 + threadIdx.x;
    if (a < A && b < B) dptr[b * A + a] = (TD)tile[threadIdx.x][i];
  }
}

// ---------------------------------------------------------------------------------------
__global__ void quantize_kernel(const void* x, DT xdt, Layout xl, void* y, DT ydt, Layout yl, Dims4 d, const float* scale, int64_t ns,
                                const float* zp, int64_t nz, float lo, float hi, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(o, yl, d);
    int64_t xi = xl == yl ? o : encode(q, xl, d);
    float v = load_as_f32(x, xdt, xi);
    float s = scale[ns > 1 ? q.c : 0];
    float z = zp ? zp[nz > 1 ? q.c : 0] : 0.f;
    float r = __fadd_rn(rintf(__fdiv_rn(v, s)), z);
    r = fminf(fmaxf(r, lo), hi);
    store_from_f32(y, ydt, o, r);
  }
}

// Per-tensor f32 -> 8-bit, same memory order on both sides: 16 elements per thread,
// four 16-byte loads and one 16-byte store.
__global__ void quantize_vec16_kernel(const float4* __restrict__ x, uint4* __restrict__ y, float scale, float zp, float lo, float hi,
                                      int64_t n16) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float4 v = x[i * 4 + j];
      float f[4] = {v.x, v.y, v.z, v.w};
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float r = __fadd_rn(rintf(__fdiv_rn(f[e], scale)), zp);
        r = fminf(fmaxf(r, lo), hi);
        w |= ((uint32_t)__float2int_rn(r) & 0xffu) << (8 * e);
      }
      packed[j] = w;
    }
    y[i] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

__global__ void dequantize_kernel(const void* x, DT xdt, Layout xl, void* y, Layout yl, Dims4 d, const float* scale, int64_t ns,
                                  const float* zp, int64_t nz, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(o, yl, d);
    int64_t xi = xl == yl ? o : encode(q, xl, d);
    float v = load_as_f32(x, xdt, xi);
    float s = scale[ns > 1 ? q.c : 0];
    float z = zp ? zp[nz > 1 ? q.c : 0] : 0.f;
    ((float*)y)[o] = __fmul_rn(__fsub_rn(v, z), s);
  }
}

// Per-tensor parameters, 8-bit lanes, same element order on both sides: four lanes per thread, a 4-byte load and
// a 16-byte store, both fully coalesced.  The byte is dropped into the mantissa of 2^23 (exact integer to float
// without the conversion pipe); (v - zp) * scale is rounded as in the generic kernel.
__global__ void dequantize_vec4_kernel(const uint32_t* __restrict__ x, bool is_signed, float4* __restrict__ y, const float* __restrict__ scale,
                                       const float* __restrict__ zp, int64_t n4) {
  const float s = scale[0], z = zp ? zp[0] : 0.f;
  const uint32_t flip = is_signed ? 0x80808080u : 0u;
  const float off = is_signed ? 8388736.0f : 8388608.0f;  // 2^23 (+ 128 for the flipped sign bit)
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t w = __ldg(x + i) ^ flip;
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float v = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 + e)), off);
      f[e] = __fmul_rn(__fsub_rn(v, z), s);
    }
    y[i] = make_float4(f[0], f[1], f[2], f[3]);
  }
}

// ---- DynamicQuantizeLinear --------------------------------------------------------------
// Order-independent min/max: floats are mapped to a monotone unsigned key so atomicMin/Max
// on integers gives the exact float extrema.
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__global__ void minmax_init_kernel(uint32_t* keys) {
  keys[0] = 0xffffffffu;  // running min key
  keys[1] = 0u;           // running max key
}

// `vec` = 0: x is not 16-byte aligned, every lane goes through the scalar loop.
__global__ void minmax_kernel(const float* __restrict__ x, int64_t n, uint32_t* keys, int vec) {
  float mn = INFINITY, mx = -INFINITY;
  int64_t n4 = vec ? n / 4 : 0;
  const float4* x4 = (const float4*)x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = x4[i];
    mn = fminf(fminf(mn, v.x), fminf(v.y, fminf(v.z, v.w)));
    mx = fmaxf(fmaxf(mx, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
  }
  for (int64_t i = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    mn = fminf(mn, x[i]);
    mx = fmaxf(mx, x[i]);
  }
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  __shared__ float smn[kThreads / 32], smx[kThreads / 32];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    smn[warp] = mn;
    smx[warp] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    mn = lane < kThreads / 32 ? smn[lane] : INFINITY;
    mx = lane < kThreads / 32 ? smx[lane] : -INFINITY;
    for (int off = 4; off > 0; off >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    if (lane == 0) {
      atomicMin(&keys[0], float_key(mn));
      atomicMax(&keys[1], float_key(mx));
    }
  }
}

// params[0] = y_scale, params[1] = y_zero_point
__global__ void dynq_params_kernel(const uint32_t* keys, float* params) {
  float max_x = fmaxf(key_float(keys[1]), 0.f);
  float min_x = fminf(key_float(keys[0]), 0.f);
  float span = (max_x == min_x) ? 1.0f : __fsub_rn(max_x, min_x);
  float y_scale = __fdiv_rn(span, 255.0f);
  float izp = __fsub_rn(0.0f, __fdiv_rn(min_x, y_scale));
  izp = fminf(fmaxf(izp, 0.f), 255.f);
  params[0] = y_scale;
  params[1] = rintf(izp);
}

__global__ void dynq_apply_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, const float* params, int64_t n) {
  float s = params[0], z = params[1];
  int64_t n4 = n / 4;  // the entry point that launches this kernel has checked the alignment of x (16) and y (4)
  const float4* x4 = (const float4*)x;
  uint32_t* y4 = (uint32_t*)y;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = x4[i];
    float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float r = __fadd_rn(rintf(__fdiv_rn(f[e], s)), z);
      r = fminf(fmaxf(r, 0.f), 255.f);
      w |= ((uint32_t)__float2int_rn(r) & 0xffu) << (8 * e);
    }
    y4[i] = w;
  }
  for (int64_t i = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float r = __fadd_rn(rintf(__fdiv_rn(x[i], s)), z);
    y[i] = (uint8_t)__float2int_rn(fminf(fmaxf(r, 0.f), 255.f));
  }
}

// The apply pass of the session path: every block derives scale and zero point from the min/max keys (the same
// operations as dynq_params_kernel, so every block gets the same two values), block 0 publishes them for the
// consumers, and the last block to finish puts the keys back to their identity values for the next call: two
// launches per DynamicQuantizeLinear instead of four.  keys[2] is the arrival counter.
__global__ void dynq_apply_fused_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, uint32_t* keys, float* params, int64_t n, int vec) {
  const float max_x = fmaxf(key_float(keys[1]), 0.f);
  const float min_x = fminf(key_float(keys[0]), 0.f);
  const float span = (max_x == min_x) ? 1.0f : __fsub_rn(max_x, min_x);
  const float s = __fdiv_rn(span, 255.0f);
  const float z = rintf(fminf(fmaxf(__fsub_rn(0.0f, __fdiv_rn(min_x, s)), 0.f), 255.f));
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    params[0] = s;
    params[1] = z;
  }
  const int64_t n4 = vec ? n / 4 : 0;  // vec = 0: x or y is not aligned for vector accesses, the scalar loop takes every lane
  const float4* x4 = (const float4*)x;
  uint32_t* y4 = (uint32_t*)y;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = x4[i];
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float r = __fadd_rn(rintf(__fdiv_rn(f[e], s)), z);
      r = fminf(fmaxf(r, 0.f), 255.f);
      w |= ((uint32_t)__float2int_rn(r) & 0xffu) << (8 * e);
    }
    y4[i] = w;
  }
  for (int64_t i = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float r = __fadd_rn(rintf(__fdiv_rn(x[i], s)), z);
    y[i] = (uint8_t)__float2int_rn(fminf(fmaxf(r, 0.f), 255.f));
  }
  __syncthreads();  // every thread of this block has read the keys
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&keys[2], 1u) == gridDim.x - 1) {
      keys[0] = 0xffffffffu;
      keys[1] = 0u;
      keys[2] = 0u;
    }
  }
}

// ---- DynamicQuantizeLinear, session path: wide passes ---------------------------------------------------
// First pass: four independent 16-byte loads per thread and iteration, one pair of atomics per block.
__global__ void __launch_bounds__(kThreads) minmax_wide_kernel(const float* __restrict__ x, int64_t n, uint32_t* keys) {
  float mn = INFINITY, mx = -INFINITY;
  const int64_t n4 = n / 4;
  const float4* x4 = (const float4*)x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t k = i + j * stride;
      v[j] = x4[k < n4 ? k : i];  // a lane past the end re-reads a valid one: neutral for both extremes
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mn = fminf(fminf(mn, v[j].x), fminf(v[j].y, fminf(v[j].z, v[j].w)));
      mx = fmaxf(fmaxf(mx, v[j].x), fmaxf(v[j].y, fmaxf(v[j].z, v[j].w)));
    }
  }
  if (blockIdx.x == 0)
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      mn = fminf(mn, x[i]);
      mx = fmaxf(mx, x[i]);
    }
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  __shared__ float smn[kThreads / 32], smx[kThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    smn[warp] = mn;
    smx[warp] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    mn = lane < kThreads / 32 ? smn[lane] : INFINITY;
    mx = lane < kThreads / 32 ? smx[lane] : -INFINITY;
    for (int off = 4; off > 0; off >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    if (lane == 0) {
      if (mn != INFINITY) atomicMin(&keys[0], float_key(mn));
      if (mx != -INFINITY) atomicMax(&keys[1], float_key(mx));
    }
  }
}

// saturate(round_ties_even(x / s) + z) as one byte.  With `safe` (s a normal number well inside the exponent
// range, so that no product below under- or overflows for |x / s| <= 256) the quotient comes from the
// reciprocal computed once per thread: q0 = x*r, one exact-remainder correction q = q0 + (x - s*q0)*r, which is
// within one unit in the last place of the correctly rounded x / s.  Rounding to an integer can then differ
// from the reference only when q lies within 2^-16 of k + 0.5; every q closer than 2^-13 to such a tie is
// recomputed with the IEEE division.  The integer rounding and the byte extraction use the 1.5 * 2^23 addend
// (an addition in round-to-nearest-even is the rounding), which keeps the conversion pipe out of the loop.
__device__ __forceinline__ uint32_t dynq_byte(float x, float s, float r, float z, bool safe) {
  const float M = 12582912.0f;
  float ri;
  if (safe) {
    const float q0 = __fmul_rn(x, r);
    const float q = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
    ri = __fsub_rn(__fadd_rn(q, M), M);
    if (fabsf(__fsub_rn(q, ri)) > 0.49987793f) ri = rintf(__fdiv_rn(x, s));
  } else {
    ri = rintf(__fdiv_rn(x, s));
  }
  const float v = fminf(fmaxf(__fadd_rn(ri, z), 0.f), 255.f);
  return __float_as_uint(__fadd_rn(v, M)) & 0xffu;
}

// Second pass: every block derives scale and zero point from the keys (the operations of dynq_params_kernel, so
// every block gets the same two values), block 0 publishes them, and the last block to finish puts the keys
// back to their identity values for the next call.  keys[2] is the arrival counter.  A warp covers 512
// consecutive lanes per iteration: four coalesced 16-byte loads and four coalesced 4-byte stores per thread.
__global__ void __launch_bounds__(kThreads) dynq_apply_wide_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, uint32_t* keys, float* params,
                                                                   int64_t n) {
  const float max_x = fmaxf(key_float(keys[1]), 0.f);
  const float min_x = fminf(key_float(keys[0]), 0.f);
  const float span = (max_x == min_x) ? 1.0f : __fsub_rn(max_x, min_x);
  const float s = __fdiv_rn(span, 255.0f);
  const float z = rintf(fminf(fmaxf(__fsub_rn(0.0f, __fdiv_rn(min_x, s)), 0.f), 255.f));
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    params[0] = s;
    params[1] = z;
  }
  const bool safe = s >= 7.8886090522101181e-31f && s <= 1.2676506002282294e+30f;  // 2^-100 .. 2^100
  const float r = safe ? __frcp_rn(s) : 0.f;
  const int64_t n4 = n / 4;
  const float4* x4 = (const float4*)x;
  uint32_t* y4 = (uint32_t*)y;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t base = ((int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * 128; base < n4; base += warps * 128) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t k = base + j * 32 + lane;
      v[j] = k < n4 ? x4[k] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t k = base + j * 32 + lane;
      const uint32_t w = dynq_byte(v[j].x, s, r, z, safe) | (dynq_byte(v[j].y, s, r, z, safe) << 8) | (dynq_byte(v[j].z, s, r, z, safe) << 16) |
                         (dynq_byte(v[j].w, s, r, z, safe) << 24);
      if (k < n4) y4[k] = w;
    }
  }
  if (blockIdx.x == 0)
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) y[i] = (uint8_t)dynq_byte(x[i], s, r, z, safe);
  __syncthreads();  // every thread of this block has read the keys
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&keys[2], 1u) == gridDim.x - 1) {
      keys[0] = 0xffffffffu;
      keys[1] = 0u;
      keys[2] = 0u;
    }
  }
}

// ---- element-wise ---------------------------------------------------------------------
__device__ __forceinline__ float apply_bin(int op, float a, float b) {
  switch (op) {
    case BIN_ADD: return __fadd_rn(a, b);
    case BIN_SUB: return __fsub_rn(a, b);
    case BIN_MUL: return __fmul_rn(a, b);
    default: return __fdiv_rn(a, b);
  }
}

__global__ void binary_kernel(const void* a, DT adt, Layout al, Dims4 ad, const void* b, DT bdt, Layout bl, Dims4 bd, void* out, DT odt,
                              Layout ol, Dims4 od, int op, int relu_after, int rtf32, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(o, ol, od);
    float av = load_as_f32(a, adt, encode_bcast(q, al, ad));
    float bv = load_as_f32(b, bdt, encode_bcast(q, bl, bd));
    float r = apply_bin(op, av, bv);
    if (relu_after) r = fmaxf(r, 0.f);
    if (rtf32) r = round_tf32(r);
    store_from_f32(out, odt, o, r);
  }
}

// Same shape, same order, f32: four elements per thread with 16-byte accesses.
__global__ void binary_vec4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out, int op,
                                   int relu_after, int rtf32, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 x = a[i], y = b[i];
    float r[4] = {apply_bin(op, x.x, y.x), apply_bin(op, x.y, y.y), apply_bin(op, x.z, y.z), apply_bin(op, x.w, y.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (relu_after) r[e] = fmaxf(r[e], 0.f);
      if (rtf32) r[e] = round_tf32(r[e]);
    }
    out[i] = make_float4(r[0], r[1], r[2], r[3]);
  }
}

// a[i] op b[i % nb]: the second operand is the trailing axes of the first (a bias row, a position table added to every
// sample), f32 in the logical order; 16-byte accesses, 32-bit index arithmetic.
__global__ void binary_suffix_vec4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out, int op, int relu_after,
                                          int rtf32, uint32_t n4, uint32_t nb4) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    const float4 x = a[i], y = __ldg(b + i % nb4);
    float r[4] = {apply_bin(op, x.x, y.x), apply_bin(op, x.y, y.y), apply_bin(op, x.z, y.z), apply_bin(op, x.w, y.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (relu_after) r[e] = fmaxf(r[e], 0.f);
      if (rtf32) r[e] = round_tf32(r[e]);
    }
    out[i] = make_float4(r[0], r[1], r[2], r[3]);
  }
}

// erf by the polynomial the reference uses (Abramowitz-Stegun 7.1.26, nn_ops/activations.rs:578), same operation order.
__device__ __forceinline__ float erf_poly(float x) {
  const float sign = x >= 0.0f ? 1.0f : -1.0f;
  x = fabsf(x);
  const float t = __frcp_rn(__fadd_rn(1.0f, __fmul_rn(0.3275911f, x)));  // the correctly rounded 1 / d, as the division gives
  float p = __fadd_rn(-1.4531521f, __fmul_rn(t, 1.0614054f));
  p = __fadd_rn(1.4214138f, __fmul_rn(t, p));
  p = __fadd_rn(-0.28449672f, __fmul_rn(t, p));
  p = __fadd_rn(0.2548296f, __fmul_rn(t, p));
  const float poly = __fmul_rn(t, p);
  return __fmul_rn(sign, __fsub_rn(1.0f, __fmul_rn(poly, expf(__fmul_rn(-x, x)))));
}

__global__ void unary_kernel(const void* x, DT xdt, void* y, DT ydt, int op, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    float v = load_as_f32(x, xdt, o);
    float r;
    switch (op) {
      case UN_RELU: r = fmaxf(v, 0.f); break;
      case UN_TANH: r = tanhf(v); break;
      case UN_SIGMOID: r = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))); break;
      case UN_SILU: r = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v))); break;
      case UN_GELU_ERF: r = __fmul_rn(__fmul_rn(v, 0.5f), __fadd_rn(1.0f, erf_poly(__fmul_rn(v, 0.70710678118654752440f)))); break;
      case UN_GELU_TANH: {
        const float inner = __fmul_rn(0.7978846f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
        r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
        break;
      }
      case UN_ERF: r = erf_poly(v); break;
      default: r = v; break;
    }
    store_from_f32(y, ydt, o, r);
  }
}

__global__ void prelu_kernel(const float* x, Layout xl, float* y, Dims4 d, const float* slope, int64_t ns, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(o, xl, d);
    float v = x[o];
    float sl = slope[ns > 1 ? q.c : 0];
    y[o] = v >= 0.f ? v : __fmul_rn(v, sl);
  }
}

// ---- pooling ----------------------------------------------------------------------------
template <typename T>
__global__ void max_pool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ y, Dims4 xd, PoolShape ps, int64_t total, T lowest) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t c = o % xd.C;
    int64_t t = o / xd.C;
    int64_t q = t % ps.Q;
    t /= ps.Q;
    int64_t p = t % ps.P;
    int64_t n = t / ps.P;
    T best = lowest;
    for (int r = 0; r < ps.kh; ++r) {
      int64_t ih = p * ps.sh + (int64_t)r * ps.dh - ps.pt;
      if (ih < 0 || ih >= xd.H) continue;
      for (int s = 0; s < ps.kw; ++s) {
        int64_t iw = q * ps.sw + (int64_t)s * ps.dw - ps.pl;
        if (iw < 0 || iw >= xd.W) continue;
        T v = x[((n * xd.H + ih) * xd.W + iw) * xd.C + c];
        if (v > best) best = v;
      }
    }
    y[o] = best;
  }
}

// Four channels of one image per thread over 8-bit lanes: every lane is dequantised as DequantizeLinear does,
// (x - zp) * scale with each operation rounded, and added in (h, w) order as the f32 kernel adds.
__global__ void global_avg_pool_nhwc_q_kernel(const uint32_t* __restrict__ x, bool is_signed, float scale, float zp, float4* __restrict__ y, Dims4 d,
                                              int rtf32) {
  const int64_t c4n = d.C / 4, total = d.N * c4n, hw = d.H * d.W;
  const uint32_t flip = is_signed ? 0x80808080u : 0u;
  const float off = is_signed ? 8388736.0f : 8388608.0f;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c4 = o % c4n, n = o / c4n;
    const uint32_t* p = x + n * hw * c4n + c4;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    int64_t i = 0;
    for (; i + 8 <= hw; i += 8) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] = __ldg(p + (i + k) * c4n) ^ flip;
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = __fsub_rn(__uint_as_float(__byte_perm(w[k], 0x4B000000u, 0x7440 + e)), off);
          sum[e] = __fadd_rn(sum[e], __fmul_rn(__fsub_rn(v, zp), scale));
        }
    }
    for (; i < hw; ++i) {
      const uint32_t w = __ldg(p + i * c4n) ^ flip;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 + e)), off);
        sum[e] = __fadd_rn(sum[e], __fmul_rn(__fsub_rn(v, zp), scale));
      }
    }
    float r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      r[e] = __fdiv_rn(sum[e], (float)hw);
      if (rtf32) r[e] = round_tf32(r[e]);
    }
    y[o] = make_float4(r[0], r[1], r[2], r[3]);
  }
}

// 16 bytes of channels per thread: four floats, or sixteen 8-bit lanes reduced with the SIMD
// byte-max instructions.  KIND 0 = f32, 1 = u8, 2 = i8.
template <int KIND>
__global__ void max_pool_nhwc_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, Dims4 xd, PoolShape ps, int64_t cvec, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t c = o % cvec;
    int64_t t = o / cvec;
    int64_t q = t % ps.Q;
    t /= ps.Q;
    int64_t p = t % ps.P;
    int64_t n = t / ps.P;
    uint4 best;
    if (KIND == 0) best = make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);  // -inf
    else if (KIND == 1) best = make_uint4(0u, 0u, 0u, 0u);
    else best = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
    for (int r = 0; r < ps.kh; ++r) {
      int64_t ih = p * ps.sh + (int64_t)r * ps.dh - ps.pt;
      if (ih < 0 || ih >= xd.H) continue;
      for (int s = 0; s < ps.kw; ++s) {
        int64_t iw = q * ps.sw + (int64_t)s * ps.dw - ps.pl;
        if (iw < 0 || iw >= xd.W) continue;
        const uint4 v = x[((n * xd.H + ih) * xd.W + iw) * cvec + c];
        if (KIND == 0) {
          // `v > best` keeps the reference's behaviour for NaN lanes (a NaN never replaces the maximum)
          if (__uint_as_float(v.x) > __uint_as_float(best.x)) best.x = v.x;
          if (__uint_as_float(v.y) > __uint_as_float(best.y)) best.y = v.y;
          if (__uint_as_float(v.z) > __uint_as_float(best.z)) best.z = v.z;
          if (__uint_as_float(v.w) > __uint_as_float(best.w)) best.w = v.w;
        } else if (KIND == 1) {
          best = make_uint4(__vmaxu4(best.x, v.x), __vmaxu4(best.y, v.y), __vmaxu4(best.z, v.z), __vmaxu4(best.w, v.w));
        } else {
          best = make_uint4(__vmaxs4(best.x, v.x), __vmaxs4(best.y, v.y), __vmaxs4(best.z, v.z), __vmaxs4(best.w, v.w));
        }
      }
    }
    y[o] = best;
  }
}

// The 3x3 / stride 2 / pad 1 pool of the ResNet front end, 16 bytes of channels per thread: the nine loads of a
// window are issued together (clamped coordinates), 32-bit index arithmetic.  KIND 0 = f32, 1 = u8, 2 = i8.
template <int KIND>
__global__ void max_pool_3x3s2_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int H, int W, int P, int Q, int cvec, int total) {
  for (int o = blockIdx.x * blockDim.x + threadIdx.x; o < total; o += gridDim.x * blockDim.x) {
    const int c = o % cvec;
    int t = o / cvec;
    const int q = t % Q;
    t /= Q;
    const int p = t % P, n = t / P;
    const int h0 = 2 * p - 1, w0 = 2 * q - 1;
    uint4 v[9];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int ih = min(max(h0 + r, 0), H - 1);
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int iw = min(max(w0 + s, 0), W - 1);
        v[3 * r + s] = __ldg(x + ((size_t)(n * H + ih) * W + iw) * cvec + c);
      }
    }
    uint4 best;
    if (KIND == 0) best = make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);  // -inf
    else if (KIND == 1) best = make_uint4(0u, 0u, 0u, 0u);
    else best = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
#pragma unroll
    for (int r = 0; r < 3; ++r) {
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        // a coordinate clamped on the low side re-reads a pixel the window holds anyway, which cannot change the
        // maximum; on the far side (odd extents) the tap lies outside the image and is dropped.  Taps are taken
        // in the reference's (r, s) order, so a NaN lane behaves as there (it never replaces the maximum).
        const bool inside = h0 + r < H && w0 + s < W && (h0 + r >= 0) && (w0 + s >= 0);
        const uint4 u = v[3 * r + s];
        if (inside) {
          if (KIND == 0) {
            if (__uint_as_float(u.x) > __uint_as_float(best.x)) best.x = u.x;
            if (__uint_as_float(u.y) > __uint_as_float(best.y)) best.y = u.y;
            if (__uint_as_float(u.z) > __uint_as_float(best.z)) best.z = u.z;
            if (__uint_as_float(u.w) > __uint_as_float(best.w)) best.w = u.w;
          } else if (KIND == 1) {
            best = make_uint4(__vmaxu4(best.x, u.x), __vmaxu4(best.y, u.y), __vmaxu4(best.z, u.z), __vmaxu4(best.w, u.w));
          } else {
            best = make_uint4(__vmaxs4(best.x, u.x), __vmaxs4(best.y, u.y), __vmaxs4(best.z, u.z), __vmaxs4(best.w, u.w));
          }
        }
      }
    }
    y[o] = best;
  }
}

// One thread per (n, c): the sum runs over the plane in (h, w) order exactly like the
// reference loop; consecutive threads read consecutive channels, so loads are coalesced.
__global__ void global_avg_pool_nhwc_kernel(const float* __restrict__ x, float* __restrict__ y, Dims4 d, int rtf32) {
  int64_t total = d.N * d.C;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t c = o % d.C, n = o / d.C;
    const float* p = x + n * d.H * d.W * d.C + c;
    float sum = 0.f;
    int64_t hw = d.H * d.W;
    // the additions keep the reference's (h, w) order; the loads of eight positions are issued together
    int64_t i = 0;
    for (; i + 8 <= hw; i += 8) {
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = p[(i + k) * d.C];
#pragma unroll
      for (int k = 0; k < 8; ++k) sum = __fadd_rn(sum, v[k]);
    }
    for (; i < hw; ++i) sum = __fadd_rn(sum, p[i * d.C]);
    float r = __fdiv_rn(sum, (float)hw);
    y[o] = rtf32 ? round_tf32(r) : r;
  }
}

// Instance norm on NHWC: one block per (n, 32-channel group); 32 lanes across channels
// (coalesced 128-byte rows), 8 warps striding over the pixels.
__global__ void instance_norm_nhwc_kernel(const float* __restrict__ x, float* __restrict__ y, Dims4 d, float eps, const float* scale_nc,
                                          const float* shift_nc, int relu, int round_tf32_flag) {
  int64_t cgroups = (d.C + 31) / 32;
  int64_t n = blockIdx.x / cgroups, cg = blockIdx.x % cgroups;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int64_t c = cg * 32 + lane;
  bool valid = c < d.C;
  int64_t hw = d.H * d.W;
  const float* px = x + n * hw * d.C + c;
  float* py = y + n * hw * d.C + c;
  __shared__ float red[32][33];
  float sum = 0.f;
  if (valid)
    for (int64_t i = warp; i < hw; i += nwarps) sum += px[i * d.C];
  red[warp][lane] = sum;
  __syncthreads();
  float tot = 0.f;
  for (int wv = 0; wv < nwarps; ++wv) tot += red[wv][lane];
  float mean = tot / (float)hw;
  __syncthreads();
  float vs = 0.f;
  if (valid)
    for (int64_t i = warp; i < hw; i += nwarps) {
      float dv = px[i * d.C] - mean;
      vs += dv * dv;
    }
  red[warp][lane] = vs;
  __syncthreads();
  tot = 0.f;
  for (int wv = 0; wv < nwarps; ++wv) tot += red[wv][lane];
  float var = tot / (float)hw;
  float inv_std = 1.0f / sqrtf(var + eps);
  float sc = 1.f, sf = 0.f;
  bool mod = scale_nc != nullptr || shift_nc != nullptr;
  if (valid && scale_nc) sc = scale_nc[n * d.C + c];
  if (valid && shift_nc) sf = shift_nc[n * d.C + c];
  if (valid)
    for (int64_t i = warp; i < hw; i += nwarps) {
      float v = (px[i * d.C] - mean) * inv_std;
      if (mod) v = v * sc + sf;  // two roundings, as the separate Mul and Add nodes (this file is built without contraction)
      if (relu) v = fmaxf(v, 0.f);
      if (round_tf32_flag) v = round_tf32(v);
      py[i * d.C] = v;
    }
}

// The same normalisation with the block's slab (all pixels x 32 channels) staged in shared memory by the first pass:
// the tensor is read from HBM once instead of three times.  32 warps stride over the pixels, four loads in flight
// each; the per-warp partial sums are added in warp order as above.
__global__ void __launch_bounds__(1024) instance_norm_nhwc_smem_kernel(const float* __restrict__ x, float* __restrict__ y, Dims4 d, float eps,
                                                                        const float* scale_nc, const float* shift_nc, int relu, int round_tf32_flag) {
  extern __shared__ float slab[];  // [pixel][32 channels]
  __shared__ float red[32][33];
  const int64_t cgroups = (d.C + 31) / 32;
  const int64_t n = blockIdx.x / cgroups, cg = blockIdx.x % cgroups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = cg * 32 + lane;
  const bool valid = c < d.C;
  const int hw = (int)(d.H * d.W);
  const float* px = x + n * hw * d.C + c;
  float* py = y + n * hw * d.C + c;
  float sum = 0.f;
  int i = warp;
  for (; i + 96 < hw; i += 128) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = valid ? px[(int64_t)(i + 32 * k) * d.C] : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      slab[(i + 32 * k) * 32 + lane] = v[k];
      sum += v[k];
    }
  }
  for (; i < hw; i += 32) {
    const float v = valid ? px[(int64_t)i * d.C] : 0.f;
    slab[i * 32 + lane] = v;
    sum += v;
  }
  red[warp][lane] = sum;
  __syncthreads();
  float tot = 0.f;
  for (int wv = 0; wv < 32; ++wv) tot += red[wv][lane];
  const float mean = tot / (float)hw;
  __syncthreads();
  float vs = 0.f;
  for (int j = warp; j < hw; j += 32) {
    const float dv = slab[j * 32 + lane] - mean;
    vs += dv * dv;
  }
  red[warp][lane] = vs;
  __syncthreads();
  tot = 0.f;
  for (int wv = 0; wv < 32; ++wv) tot += red[wv][lane];
  const float var = tot / (float)hw;
  const float inv_std = 1.0f / sqrtf(var + eps);
  float sc = 1.f, sf = 0.f;
  const bool mod = scale_nc != nullptr || shift_nc != nullptr;
  if (valid && scale_nc) sc = scale_nc[n * d.C + c];
  if (valid && shift_nc) sf = shift_nc[n * d.C + c];
  if (valid)
    for (int j = warp; j < hw; j += 32) {
      float v = (slab[j * 32 + lane] - mean) * inv_std;
      if (mod) v = v * sc + sf;  // two roundings, as the separate Mul and Add nodes (this file is built without contraction)
      if (relu) v = fmaxf(v, 0.f);
      if (round_tf32_flag) v = round_tf32(v);
      py[(int64_t)j * d.C] = v;
    }
}

// ---- resize / pad / concat --------------------------------------------------------------
__device__ __forceinline__ float src_coord(int coord, int64_t o, float scale, int64_t in_size, int64_t out_size) {
  switch (coord) {
    case 2: return __fdiv_rn((float)o, scale);
    case 3: return out_size <= 1 ? 0.f : __fdiv_rn(__fmul_rn((float)o, (float)(in_size - 1)), (float)(out_size - 1));
    case 1: return out_size > 1 ? __fsub_rn(__fdiv_rn(__fadd_rn((float)o, 0.5f), scale), 0.5f) : 0.f;
    default: return __fsub_rn(__fdiv_rn(__fadd_rn((float)o, 0.5f), scale), 0.5f);
  }
}
__device__ __forceinline__ int64_t nearest_index(int rule, float s, int64_t in_size) {
  float r;
  switch (rule) {
    case 1: r = floorf(s); break;
    case 2: r = ceilf(s); break;
    case 3: r = floorf(__fadd_rn(s, 0.5f)); break;
    default: r = ceilf(__fsub_rn(s, 0.5f)); break;
  }
  int64_t i = (int64_t)r;
  return i < 0 ? 0 : (i > in_size - 1 ? in_size - 1 : i);
}

__global__ void resize_nhwc_kernel(const float* __restrict__ x, float* __restrict__ y, Dims4 xd, Dims4 yd, int mode, int coord, int rule,
                                   float sh, float sw, int64_t total, int rtf32) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t c = o % yd.C;
    int64_t t = o / yd.C;
    int64_t ox = t % yd.W;
    t /= yd.W;
    int64_t oy = t % yd.H;
    int64_t n = t / yd.H;
    float sy = src_coord(coord, oy, sh, xd.H, yd.H), sx = src_coord(coord, ox, sw, xd.W, yd.W);
    const float* base = x + n * xd.H * xd.W * xd.C + c;
    if (mode == 0) {
      y[o] = base[(nearest_index(rule, sy, xd.H) * xd.W + nearest_index(rule, sx, xd.W)) * xd.C];
    } else {
      float cy = fminf(fmaxf(sy, 0.f), (float)(xd.H - 1)), cx = fminf(fmaxf(sx, 0.f), (float)(xd.W - 1));
      int64_t y0 = (int64_t)floorf(cy), x0 = (int64_t)floorf(cx);
      int64_t y1 = y0 + 1 < xd.H ? y0 + 1 : xd.H - 1, x1 = x0 + 1 < xd.W ? x0 + 1 : xd.W - 1;
      float fy = __fsub_rn(cy, (float)y0), fx = __fsub_rn(cx, (float)x0);
      float v00 = base[(y0 * xd.W + x0) * xd.C], v01 = base[(y0 * xd.W + x1) * xd.C];
      float v10 = base[(y1 * xd.W + x0) * xd.C], v11 = base[(y1 * xd.W + x1) * xd.C];
      float top = __fadd_rn(__fmul_rn(v00, __fsub_rn(1.f, fx)), __fmul_rn(v01, fx));
      float bot = __fadd_rn(__fmul_rn(v10, __fsub_rn(1.f, fx)), __fmul_rn(v11, fx));
      const float r = __fadd_rn(__fmul_rn(top, __fsub_rn(1.f, fy)), __fmul_rn(bot, fy));
      y[o] = rtf32 ? round_tf32(r) : r;
    }
  }
}

// Four channels per thread (NHWC f32, C % 4 == 0): the same arithmetic per lane as the scalar kernel.
template <typename I>  // index type: 32-bit divisions where the tensor allows them
__global__ void resize_nhwc_vec4_kernel(const float4* __restrict__ x, float4* __restrict__ y, Dims4 xd, Dims4 yd, int mode, int coord, int rule,
                                        float sh, float sw, int64_t total4, int rtf32) {
  const I c4n = (I)(yd.C / 4), yW = (I)yd.W, yH = (I)yd.H;
  for (I o = (I)(blockIdx.x * (int64_t)blockDim.x + threadIdx.x); o < (I)total4; o += (I)((int64_t)gridDim.x * blockDim.x)) {
    const I c4 = o % c4n;
    I t = o / c4n;
    const I ox = t % yW;
    t /= yW;
    const I oy = t % yH;
    const int64_t n = t / yH;
    const float sy = src_coord(coord, oy, sh, xd.H, yd.H), sx = src_coord(coord, ox, sw, xd.W, yd.W);
    const float4* base = x + n * xd.H * xd.W * c4n + c4;
    if (mode == 0) {
      y[o] = base[(nearest_index(rule, sy, xd.H) * xd.W + nearest_index(rule, sx, xd.W)) * c4n];
    } else {
      const float cy = fminf(fmaxf(sy, 0.f), (float)(xd.H - 1)), cx = fminf(fmaxf(sx, 0.f), (float)(xd.W - 1));
      const int64_t y0 = (int64_t)floorf(cy), x0 = (int64_t)floorf(cx);
      const int64_t y1 = y0 + 1 < xd.H ? y0 + 1 : xd.H - 1, x1 = x0 + 1 < xd.W ? x0 + 1 : xd.W - 1;
      const float fy = __fsub_rn(cy, (float)y0), fx = __fsub_rn(cx, (float)x0);
      const float gx = __fsub_rn(1.f, fx), gy = __fsub_rn(1.f, fy);
      const float4 v00 = base[(y0 * xd.W + x0) * c4n], v01 = base[(y0 * xd.W + x1) * c4n];
      const float4 v10 = base[(y1 * xd.W + x0) * c4n], v11 = base[(y1 * xd.W + x1) * c4n];
      float4 r;
#define OXB_LERP(f)                                                                          \
  {                                                                                          \
    const float top = __fadd_rn(__fmul_rn(v00.f, gx), __fmul_rn(v01.f, fx));                 \
    const float bot = __fadd_rn(__fmul_rn(v10.f, gx), __fmul_rn(v11.f, fx));                 \
    r.f = __fadd_rn(__fmul_rn(top, gy), __fmul_rn(bot, fy));                                 \
  }
      OXB_LERP(x) OXB_LERP(y) OXB_LERP(z) OXB_LERP(w)
#undef OXB_LERP
      if (rtf32) r = make_float4(round_tf32(r.x), round_tf32(r.y), round_tf32(r.z), round_tf32(r.w));  // the lanes feed a TF32 product
      y[o] = r;
    }
  }
}

__device__ __forceinline__ int64_t pad_src(int64_t idx, int64_t ext, int mode, bool& outside) {
  if (idx >= 0 && idx < ext) return idx;
  if (mode == 0) {
    outside = true;
    return 0;
  }
  if (mode == 2) return idx < 0 ? 0 : ext - 1;
  return idx < 0 ? -idx : 2 * (ext - 1) - idx;
}

__global__ void pad_kernel(const void* x, void* y, DT dt, Layout L, Dims4 xd, Dims4 yd, int mode, float value, int pn, int pc, int ph, int pw,
                           int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(o, L, yd);
    bool outside = false;
    Coord sq;
    sq.n = pad_src(q.n - pn, xd.N, mode, outside);
    sq.c = pad_src(q.c - pc, xd.C, mode, outside);
    sq.h = pad_src(q.h - ph, xd.H, mode, outside);
    sq.w = pad_src(q.w - pw, xd.W, mode, outside);
    float v = outside ? value : load_as_f32(x, dt, encode(sq, L, xd));
    store_from_f32(y, dt, o, v);
  }
}

// Spatial padding of an NHWC tensor in 16-byte pieces (any storage type whose pixel is a multiple of 16 bytes).
template <typename I>  // index type: 32-bit divisions where the tensor allows them
__global__ void pad_nhwc_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, Dims4 xd, Dims4 yd, int64_t vec_per_pixel, int mode, uint4 fill,
                                    int ph, int pw, int64_t total) {
  const I vpp = (I)vec_per_pixel, yW = (I)yd.W, yH = (I)yd.H;
  for (I o = (I)(blockIdx.x * (int64_t)blockDim.x + threadIdx.x); o < (I)total; o += (I)((int64_t)gridDim.x * blockDim.x)) {
    const int64_t v = o % vpp;
    I t = o / vpp;
    const int64_t ow = t % yW;
    t /= yW;
    const int64_t oh = t % yH;
    const int64_t n = t / yH;
    bool outside = false;
    const int64_t ih = pad_src(oh - ph, xd.H, mode, outside), iw = pad_src(ow - pw, xd.W, mode, outside);
    y[o] = outside ? fill : x[((n * xd.H + ih) * xd.W + iw) * vec_per_pixel + v];
  }
}

__global__ void concat_kernel(const void* x, void* y, DT dt, Layout L, Dims4 xd, Dims4 yd, int axis, int64_t offset, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    Coord q = decode(i, L, xd);
    if (axis == 0) q.n += offset;
    else if (axis == 1) q.c += offset;
    else if (axis == 2) q.h += offset;
    else q.w += offset;
    int64_t o = encode(q, L, yd);
    size_t es = dt == DT::F32 || dt == DT::I32 ? 4 : (dt == DT::I16 ? 2 : 1);
    if (es == 4) ((uint32_t*)y)[o] = ((const uint32_t*)x)[i];
    else if (es == 2) ((uint16_t*)y)[o] = ((const uint16_t*)x)[i];
    else ((uint8_t*)y)[o] = ((const uint8_t*)x)[i];
  }
}

__device__ __forceinline__ float lane8(uint32_t word, int e, bool is_signed) {
  uint32_t b = (word >> (8 * e)) & 0xffu;
  return is_signed ? (float)(int)(int8_t)b : (float)b;
}

__device__ __forceinline__ uint32_t residual_one(float av, float bv, const ResidualParams& rp) {
  float va = __fmul_rn(__fsub_rn(av, rp.a_zp), rp.a_scale);
  float vb = __fmul_rn(__fsub_rn(bv, rp.b_zp), rp.b_scale);
  float sum = __fadd_rn(va, vb);
  if (rp.relu) sum = fmaxf(sum, 0.f);
  float q = __fadd_rn(rintf(__fdiv_rn(sum, rp.y_scale)), rp.y_zp);
  q = fminf(fmaxf(q, rp.lo), rp.hi);
  return (uint32_t)__float2int_rn(q) & 0xffu;
}

// The same lane without the conversion and reciprocal units, for parameters that
// residual_requant_prepare() has proven: the byte is dropped into the mantissa of 2^23 (so that
// `bits - (2^23 + zp)` is the exact integer difference), the quotient is one multiply by the
// rounded reciprocal plus one remainder correction, and rounding to the nearest-even integer is an
// addition of 1.5 * 2^23.  `off_a`/`off_b` are 2^23 + zero point (+128 for signed storage, whose
// bytes arrive with the sign bit flipped).
__device__ __forceinline__ float residual_fast(uint32_t a_bits, uint32_t b_bits, float off_a, float off_b, const ResidualParams& rp) {
  const float va = __fmul_rn(__fsub_rn(__uint_as_float(a_bits), off_a), rp.a_scale);
  const float vb = __fmul_rn(__fsub_rn(__uint_as_float(b_bits), off_b), rp.b_scale);
  float sum = __fadd_rn(va, vb);
  if (rp.relu) sum = fmaxf(sum, 0.f);
  const float q0 = __fmul_rn(sum, rp.y_rcp);
  const float q = __fmaf_rn(__fmaf_rn(-q0, rp.y_scale, sum), rp.y_rcp, q0);
  const float t = __fadd_rn(__fadd_rn(q, 12582912.0f), rp.y_zp);
  return fminf(fmaxf(t, 12582912.0f + rp.lo), 12582912.0f + rp.hi);  // the lane is the low byte of these bits
}

// 16 lanes per thread: two 16-byte loads, one 16-byte store.
// ---- the same lane, two at a time (proven_fast == 2) ------------------------------------------------------------
// f32x2 instructions give the IEEE result of each lane with half the issue slots; the ReLU is folded into the lower
// clamp bound (the quotient by a positive scale and the rounding are monotone and map 0 to 0, so
// max(round(sum / s), 0) + zp == round(max(sum, 0) / s) + zp); and because 1.5 * 2^23 has sixteen zero low bits, the
// low half-word of t = (q + 1.5 * 2^23) + zp is the rounded result itself as an int16, so two results are clamped
// with one packed max and one packed min.  residual_requant_prepare() evaluates exactly this formula for all
// 256 x 256 input pairs and enables it only when every pair gives the reference's lane and stays inside int16.
struct F2 {
  float x, y;
};
__device__ __forceinline__ F2 add2(F2 a, F2 b) {
  uint64_t ra, rb, rd;
  F2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ F2 mul2(F2 a, F2 b) {
  uint64_t ra, rb, rd;
  F2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ F2 fma2(F2 a, F2 b, F2 c) {
  uint64_t ra, rb, rc, rd;
  F2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
// Two lanes (bytes e and e + 1 of the words wa, wb): returns the two clamped results as packed int16.
__device__ __forceinline__ uint32_t residual_pair(uint32_t wa, uint32_t wb, int e, F2 noff_a, F2 noff_b, F2 sa, F2 sb, F2 rcp, F2 nys, F2 magic, F2 zp,
                                                  uint32_t lo2, uint32_t hi2) {
  const F2 abits = {__uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7440 + e)), __uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7441 + e))};
  const F2 bbits = {__uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7440 + e)), __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7441 + e))};
  // The two dequantising products are scalar __fmul_rn: on this toolchain a packed multiply whose result feeds a
  // packed add came out as if fused (5 * 0.02f + 0.05f gave 0.15f, not 0.14999999f), which moves exact ties.
  const F2 da = add2(abits, noff_a), db = add2(bbits, noff_b);
  const F2 va = {__fmul_rn(da.x, sa.x), __fmul_rn(da.y, sa.y)}, vb = {__fmul_rn(db.x, sb.x), __fmul_rn(db.y, sb.y)};
  const F2 sum = add2(va, vb);
  const F2 q0 = mul2(sum, rcp);
  const F2 q = fma2(fma2(q0, nys, sum), rcp, q0);
  const F2 t = add2(add2(q, magic), zp);
  const uint32_t p = __byte_perm(__float_as_uint(t.x), __float_as_uint(t.y), 0x5410);
  return __vmins2(__vmaxs2(p, lo2), hi2);
}

template <int MODE>
__device__ __forceinline__ uint4 residual_vec(const uint4 av, const uint4 bv, bool a_signed, bool b_signed, float off_a, float off_b, uint32_t flip_a,
                                              uint32_t flip_b, const ResidualParams& rp) {
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
    uint32_t out[4];
    if (MODE == 2) {
      const float lo_eff = rp.relu ? fmaxf(rp.lo, rp.y_zp) : rp.lo;
      const uint32_t lo2 = ((uint32_t)(int)lo_eff & 0xffffu) * 0x00010001u, hi2 = ((uint32_t)(int)rp.hi & 0xffffu) * 0x00010001u;
      const F2 noff_a = {-off_a, -off_a}, noff_b = {-off_b, -off_b}, sa = {rp.a_scale, rp.a_scale}, sb = {rp.b_scale, rp.b_scale};
      const F2 rcp = {rp.y_rcp, rp.y_rcp}, nys = {-rp.y_scale, -rp.y_scale}, magic = {12582912.0f, 12582912.0f}, zp = {rp.y_zp, rp.y_zp};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t wa = aw[j] ^ flip_a, wb = bw[j] ^ flip_b;
        const uint32_t p01 = residual_pair(wa, wb, 0, noff_a, noff_b, sa, sb, rcp, nys, magic, zp, lo2, hi2);
        const uint32_t p23 = residual_pair(wa, wb, 2, noff_a, noff_b, sa, sb, rcp, nys, magic, zp, lo2, hi2);
        out[j] = __byte_perm(p01, p23, 0x6420);
      }
      return make_uint4(out[0], out[1], out[2], out[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (MODE == 1) {
        const uint32_t wa = aw[j] ^ flip_a, wb = bw[j] ^ flip_b;
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          r[e] = __float_as_uint(residual_fast(__byte_perm(wa, 0x4B000000u, 0x7440 + e), __byte_perm(wb, 0x4B000000u, 0x7440 + e), off_a, off_b, rp));
        out[j] = __byte_perm(__byte_perm(r[0], r[1], 0x0040), __byte_perm(r[2], r[3], 0x0040), 0x5410);
      } else {
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) w |= residual_one(lane8(aw[j], e, a_signed), lane8(bw[j], e, b_signed), rp) << (8 * e);
        out[j] = w;
      }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// 16 lanes per thread and iteration: two 16-byte loads, one 16-byte store.  Two vectors per iteration (four loads
// in flight) were measured and are slower (4.46 against 4.65 TB/s on 822 MB operands): the grid already keeps
// enough bytes in flight, and the longer body costs occupancy.
template <int MODE>
__global__ void residual_requant_kernel(const uint4* __restrict__ a, bool a_signed, const uint4* __restrict__ b, bool b_signed, uint4* __restrict__ y,
                                        int64_t n16, ResidualParams rp) {
  const float off_a = 8388608.0f + rp.a_zp + (a_signed ? 128.f : 0.f), off_b = 8388608.0f + rp.b_zp + (b_signed ? 128.f : 0.f);
  const uint32_t flip_a = a_signed ? 0x80808080u : 0u, flip_b = b_signed ? 0x80808080u : 0u;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = residual_vec<MODE>(__ldcs(a + i), __ldcs(b + i), a_signed, b_signed, off_a, off_b, flip_a, flip_b, rp);
}

__global__ void residual_requant_tail_kernel(const uint8_t* a, bool a_signed, const uint8_t* b, bool b_signed, uint8_t* y, int64_t begin, int64_t n,
                                             ResidualParams rp) {
  for (int64_t i = begin + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float av = a_signed ? (float)(int8_t)a[i] : (float)a[i];
    float bv = b_signed ? (float)(int8_t)b[i] : (float)b[i];
    y[i] = (uint8_t)residual_one(av, bv, rp);
  }
}

// Four consecutive packed channels per thread, written as one 4-byte or 16-byte store.
__global__ void s2d_pack_kernel(const void* src, DT sdt, Layout sl, Dims4 d, void* dst, DT ddt, int c_pad, int sub, int64_t total4) {
  const int64_t H2 = d.H / 2, W2 = d.W / 2;
  const int c4n = c_pad / 4;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total4; o += (int64_t)gridDim.x * blockDim.x) {
    const int cq = (int)(o % c4n);
    int64_t t = o / c4n;
    const int64_t x = t % W2;
    t /= W2;
    const int64_t y = t % H2;
    const int64_t n = t / H2;
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int cp = cq * 4 + e;
      v[e] = 0.f;
      if (cp < 4 * d.C) {
        const int blk = cp / (int)d.C;
        Coord q;
        q.n = n;
        q.c = cp - blk * (int)d.C;
        q.h = 2 * y + (blk >> 1);
        q.w = 2 * x + (blk & 1);
        v[e] = load_as_f32(src, sdt, encode(q, sl, d)) - (float)sub;
      }
    }
    if (ddt == DT::F32) {
      ((float4*)dst)[o] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = ddt == DT::U8 ? 0.f : -128.f, hi = ddt == DT::U8 ? 255.f : 127.f;
        w |= ((uint32_t)__float2int_rn(fminf(fmaxf(v[e], lo), hi)) & 0xffu) << (8 * e);
      }
      ((uint32_t*)dst)[o] = w;
    }
  }
}

// One packed pixel (16 lanes) per thread.
// Row pairs (8-bit destinations, `pair_top` >= 0): the destination is [N][rows_phys][wp][32] -- physical row j holds
// the packed block of image row j - pair_top in lanes 0..15 and that of image row j - pair_top + 1 in lanes 16..31
// (zeros where there is no such row: the vertical padding is physical) -- so that one window of S2p pixels covers two
// filter rows in 128 contiguous bytes.  A thread makes the block of one (row, pixel) and stores it in both places;
// the row index runs over rows_phys + 1 values so that every half of every physical row is written exactly once.
__device__ __forceinline__ void s2d_store_pair(void* dst, uint4 block, int64_t n, int64_t jp, int64_t xw, int rows_phys, int wp) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  if (jp < rows_phys) d4[((n * rows_phys + jp) * wp + xw) * 2] = block;
  if (jp >= 1) d4[((n * rows_phys + jp - 1) * wp + xw) * 2 + 1] = block;
}

__global__ void s2d_window_pack_kernel(const void* src, DT sdt, Layout sl, Dims4 d, void* dst, DT ddt, int pad_left, int wp, int sub, S2dQuant q,
                                       int64_t total, int pair_top, int rows_phys) {
  const int64_t H2 = d.H / 2, W2 = d.W / 2;
  const int c4 = 4 * (int)d.C;
  const int64_t rows = pair_top >= 0 ? rows_phys + 1 : H2;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t xw = o % wp;
    int64_t t = o / wp;
    const int64_t jp = t % rows;
    const int64_t y = pair_top >= 0 ? jp - pair_top : jp;
    const int64_t n = t / rows;
    const int64_t x2 = xw - pad_left;
    float v[16];
#pragma unroll
    for (int cp = 0; cp < 16; ++cp) {
      v[cp] = 0.f;
      if (cp < c4 && x2 >= 0 && x2 < W2 && y >= 0 && y < H2) {
        const int blk = cp / (int)d.C;
        Coord qd;
        qd.n = n;
        qd.c = cp - blk * (int)d.C;
        qd.h = 2 * y + (blk >> 1);
        qd.w = 2 * x2 + (blk & 1);
        float f = load_as_f32(src, sdt, encode(qd, sl, d));
        if (q.quantize) f = fminf(fmaxf(__fadd_rn(rintf(__fdiv_rn(f, q.scale)), q.zp), q.lo), q.hi);
        v[cp] = f - (float)sub;
      }
    }
    if (ddt == DT::F32) {
#pragma unroll
      for (int j = 0; j < 4; ++j) ((float4*)dst)[o * 4 + j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      const float lo = ddt == DT::U8 ? 0.f : -128.f, hi = ddt == DT::U8 ? 255.f : 127.f;
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        w[j] = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) w[j] |= ((uint32_t)__float2int_rn(fminf(fmaxf(v[4 * j + e], lo), hi)) & 0xffu) << (8 * e);
      }
      if (pair_top >= 0) s2d_store_pair(dst, make_uint4(w[0], w[1], w[2], w[3]), n, jp, xw, rows_phys, wp);
      else ((uint4*)dst)[o] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// round_ties_even(x / s) without the division on the common path: the quotient from the correctly rounded
// reciprocal r with one exact-remainder correction is within one unit in the last place of the IEEE quotient
// (s a normal number in 2^-100 .. 2^100, |q| < 1024, so that a unit is at most 2^-14); only a q closer than
// 2^-13 to a tie k + 1/2 could round differently, and those lanes, like every lane outside the proven range,
// take the division.
__device__ __forceinline__ float quotient_rint(float x, float s, float r, bool safe) {
  if (safe) {
    const float q0 = __fmul_rn(x, r);
    const float q = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
    if (fabsf(q) < 1024.0f) {
      const float ri = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
      if (fabsf(__fsub_rn(q, ri)) <= 0.49987793f) return ri;
    }
  }
  return rintf(__fdiv_rn(x, s));
}

// The same packing for the common source: f32 NCHW with an even width.  The two horizontally adjacent pixels of
// a 2x2 block come from one 8-byte load, and consecutive threads read consecutive blocks (fully coalesced).
template <int C>
__global__ void s2d_window_pack_nchw_f32_kernel(const float* __restrict__ src, Dims4 d, void* dst, DT ddt, int pad_left, int wp, int sub, S2dQuant q,
                                                float rcp, bool safe, int64_t total, int pair_top, int rows_phys) {
  const int64_t H2 = d.H / 2, W2 = d.W / 2;
  const int64_t rows = pair_top >= 0 ? rows_phys + 1 : H2;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t xw = o % wp;
    int64_t t = o / wp;
    const int64_t jp = t % rows;
    const int64_t y = pair_top >= 0 ? jp - pair_top : jp;
    const int64_t n = t / rows;
    const int64_t x2 = xw - pad_left;
    float v[16];
#pragma unroll
    for (int cp = 0; cp < 16; ++cp) v[cp] = 0.f;
    if (x2 >= 0 && x2 < W2 && y >= 0 && y < H2) {
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const float* plane = src + ((n * C + c) * d.H + 2 * y) * d.W + 2 * x2;
        const float2 top = __ldg(reinterpret_cast<const float2*>(plane));
        const float2 bot = __ldg(reinterpret_cast<const float2*>(plane + d.W));
        v[0 * C + c] = top.x;
        v[1 * C + c] = top.y;
        v[2 * C + c] = bot.x;
        v[3 * C + c] = bot.y;
      }
#pragma unroll
      for (int cp = 0; cp < 4 * C; ++cp) {
        float f = v[cp];
        if (q.quantize) f = fminf(fmaxf(__fadd_rn(quotient_rint(f, q.scale, rcp, safe), q.zp), q.lo), q.hi);
        v[cp] = f - (float)sub;
      }
    }
    if (ddt == DT::F32) {
#pragma unroll
      for (int j = 0; j < 4; ++j) ((float4*)dst)[o * 4 + j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      const float lo = ddt == DT::U8 ? 0.f : -128.f, hi = ddt == DT::U8 ? 255.f : 127.f;
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        w[j] = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          w[j] |= (__float_as_uint(__fadd_rn(fminf(fmaxf(v[4 * j + e], lo), hi), 12582912.0f)) & 0xffu) << (8 * e);
      }
      if (pair_top >= 0) s2d_store_pair(dst, make_uint4(w[0], w[1], w[2], w[3]), n, jp, xw, rows_phys, wp);
      else ((uint4*)dst)[o] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// The same packing for an 8-bit NCHW source (a graph input declared uint8 / int8) into an 8-bit destination: the
// two horizontally adjacent pixels of a 2x2 block are one 2-byte load, consecutive threads read consecutive blocks.
template <int C, bool SIGNED>
__global__ void s2d_window_pack_nchw_q8_kernel(const uint8_t* __restrict__ src, Dims4 d, void* dst, DT ddt, int pad_left, int wp, int sub, int64_t total,
                                               int pair_top, int rows_phys) {
  const int64_t H2 = d.H / 2, W2 = d.W / 2;
  const int64_t rows = pair_top >= 0 ? rows_phys + 1 : H2;
  const int lo = ddt == DT::U8 ? 0 : -128, hi = ddt == DT::U8 ? 255 : 127;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t xw = o % wp;
    int64_t t = o / wp;
    const int64_t jp = t % rows;
    const int64_t y = pair_top >= 0 ? jp - pair_top : jp;
    const int64_t n = t / rows;
    const int64_t x2 = xw - pad_left;
    int v[16];
#pragma unroll
    for (int cp = 0; cp < 16; ++cp) v[cp] = 0;
    if (x2 >= 0 && x2 < W2 && y >= 0 && y < H2) {
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const uint8_t* plane = src + ((n * C + c) * d.H + 2 * y) * d.W + 2 * x2;
        const uint32_t top = __ldg(reinterpret_cast<const uint16_t*>(plane));
        const uint32_t bot = __ldg(reinterpret_cast<const uint16_t*>(plane + d.W));
        const uint32_t b[4] = {top & 0xffu, top >> 8, bot & 0xffu, bot >> 8};
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k * C + c] = min(max((SIGNED ? (int)(int8_t)b[k] : (int)b[k]) - sub, lo), hi);
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = ((uint32_t)v[4 * j] & 0xffu) | (((uint32_t)v[4 * j + 1] & 0xffu) << 8) | (((uint32_t)v[4 * j + 2] & 0xffu) << 16) | (((uint32_t)v[4 * j + 3] & 0xffu) << 24);
    if (pair_top >= 0) s2d_store_pair(dst, make_uint4(w[0], w[1], w[2], w[3]), n, jp, xw, rows_phys, wp);
    else ((uint4*)dst)[o] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// y = x[start0 : start0 + Y0, start1 : ..., ...] over up to four logical (row-major) axes, unit steps.
__global__ void slice_kernel(const void* x, void* y, int es, Dims4 xd, Dims4 yd, Dims4 start, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = o;
    const int64_t i3 = t % yd.W;
    t /= yd.W;
    const int64_t i2 = t % yd.H;
    t /= yd.H;
    const int64_t i1 = t % yd.C;
    const int64_t i0 = t / yd.C;
    const int64_t src = (((i0 + start.N) * xd.C + (i1 + start.C)) * xd.H + (i2 + start.H)) * xd.W + (i3 + start.W);
    if (es == 4) ((uint32_t*)y)[o] = ((const uint32_t*)x)[src];
    else if (es == 2) ((uint16_t*)y)[o] = ((const uint16_t*)x)[src];
    else ((uint8_t*)y)[o] = ((const uint8_t*)x)[src];
  }
}

// Row-window packing without space-to-depth (stride-1 convolutions over up to four f32 channels):
// dst is [N][H][wp][4], four lanes per pixel (C values, then zeros), `pad_left` zero pixels in front of
// every row and zeros behind it.  One pixel (16 bytes) per thread.
__global__ void window_pack_f32_kernel(const float* __restrict__ src, Layout sl, Dims4 d, float4* __restrict__ dst, int pad_left, int wp,
                                       int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t xw = o % wp;
    int64_t t = o / wp;
    const int64_t y = t % d.H;
    const int64_t n = t / d.H;
    const int64_t x = xw - pad_left;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (x >= 0 && x < d.W) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c < d.C) {
          Coord q;
          q.n = n, q.c = c, q.h = y, q.w = x;
          v[c] = src[encode(q, sl, d)];
        }
    }
    dst[o] = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// ---- transformer glue ---------------------------------------------------------------------
// Gather along axis 0 of a [rows, inner] table: one output row per index lane (an f32 lane holding
// an integer; negative values count from the end).  An index outside the table records code 20.
__global__ void gather_rows_kernel(const float* __restrict__ table, const float* __restrict__ idx, float* __restrict__ out, int64_t n_idx, int64_t rows,
                                   int64_t inner, int* err) {
  const int64_t total = n_idx * inner;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = o / inner, j = o - i * inner;
    long long r = (long long)idx[i];
    if (r < 0) r += rows;
    if (r < 0 || r >= rows) {
      if (j == 0) atomicExch(err, 20);
      out[o] = 0.f;
      continue;
    }
    out[o] = table[r * inner + j];
  }
}

// Permutation of up to four logical axes: yd is the output shape, xstride[d] the input stride of output axis d.
__global__ void transpose_perm_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, Dims4 yd, Dims4 xstride, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = o;
    const int64_t i3 = t % yd.W;
    t /= yd.W;
    const int64_t i2 = t % yd.H;
    t /= yd.H;
    const int64_t i1 = t % yd.C;
    const int64_t i0 = t / yd.C;
    y[o] = x[i0 * xstride.N + i1 * xstride.C + i2 * xstride.H + i3 * xstride.W];
  }
}

// The same permutation when the innermost axis stays innermost (head split / merge of attention tensors): 16-byte
// pieces of the inner rows, 32-bit index arithmetic.
__global__ void transpose_perm_vec4_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, uint32_t d1, uint32_t d2, uint32_t w4, uint32_t s0, uint32_t s1,
                                           uint32_t s2, uint32_t total4) {
  for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total4; o += gridDim.x * blockDim.x) {
    uint32_t t = o;
    const uint32_t i3 = t % w4;
    t /= w4;
    const uint32_t i2 = t % d2;
    t /= d2;
    const uint32_t i1 = t % d1;
    const uint32_t i0 = t / d1;
    y[o] = x[i0 * s0 + i1 * s1 + i2 * s2 + i3];
  }
}

// The same permutation when the input's contiguous axis becomes the output's second-to-last one (V -> V^T per head):
// 32 x 32 tiles through shared memory, 128-byte reads along the input rows and 128-byte writes along the output rows.
__global__ void transpose_tiled_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, Dims4 yd, Dims4 xs, int64_t blocks) {
  __shared__ uint32_t tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 256 threads: 8 rows of a tile per pass
  const int64_t th = (yd.H + 31) / 32, tw = (yd.W + 31) / 32;
  for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
    int64_t t = b;
    const int64_t w0 = (t % tw) * 32;
    t /= tw;
    const int64_t h0 = (t % th) * 32;
    t /= th;
    const int64_t i1 = t % yd.C, i0 = t / yd.C;
    const uint32_t* src = x + i0 * xs.N + i1 * xs.C;
    uint32_t* dst = y + (i0 * yd.C + i1) * yd.H * yd.W;
#pragma unroll
    for (int k = ty; k < 32; k += 8)
      if (h0 + tx < yd.H && w0 + k < yd.W) tile[k][tx] = src[(h0 + tx) + (w0 + k) * xs.W];
    __syncthreads();
#pragma unroll
    for (int k = ty; k < 32; k += 8)
      if (h0 + k < yd.H && w0 + tx < yd.W) dst[(h0 + k) * yd.W + (w0 + tx)] = tile[tx][k];
    __syncthreads();
  }
}

// The same transposition for inner extents that are multiples of four on both sides: a block moves a tile of
// 32 output rows (the input's contiguous axis) x 128 output columns with 16-byte loads along the input rows and
// 16-byte stores along the output rows.
__global__ void transpose_tiled_vec4_kernel(const float* __restrict__ x, float* __restrict__ y, Dims4 yd, Dims4 xs, int64_t blocks) {
  __shared__ float tile[128][33];  // [output column][output row]
  const int64_t th = (yd.H + 31) / 32, tw = (yd.W + 127) / 128;
  for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
    int64_t t = b;
    const int64_t w0 = (t % tw) * 128;
    t /= tw;
    const int64_t h0 = (t % th) * 32;
    t /= th;
    const int64_t i1 = t % yd.C, i0 = t / yd.C;
    const float* src = x + i0 * xs.N + i1 * xs.C;
    float* dst = y + (i0 * yd.C + i1) * yd.H * yd.W;
    // loads: 8 threads cover the 32 contiguous input lanes (output rows h0..h0+31) of one output column
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int col = (int)(threadIdx.x >> 3) + 32 * k, h4 = (int)(threadIdx.x & 7) * 4;
      if (w0 + col < yd.W && h0 + h4 < yd.H) {
        const float4 v = *reinterpret_cast<const float4*>(src + (w0 + col) * xs.W + h0 + h4);
        tile[col][h4] = v.x, tile[col][h4 + 1] = v.y, tile[col][h4 + 2] = v.z, tile[col][h4 + 3] = v.w;
      }
    }
    __syncthreads();
    // stores: 32 threads cover the 128 contiguous output columns of one output row
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int row = (int)(threadIdx.x >> 5) + 8 * k, c4 = (int)(threadIdx.x & 31) * 4;
      if (h0 + row < yd.H && w0 + c4 < yd.W)
        *reinterpret_cast<float4*>(dst + (h0 + row) * yd.W + w0 + c4) = make_float4(tile[c4][row], tile[c4 + 1][row], tile[c4 + 2][row], tile[c4 + 3][row]);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Softmax over the last axis, one warp per row: max, exp(v - max), sum, multiply by 1 / sum
// (nn/normalization.rs softmax_into; the sums are reassociated across lanes: float tolerance).
__global__ void softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t rows, int64_t n, const float* __restrict__ scale,
                                    const float* __restrict__ mask, int64_t rows_per_mask, int round_tf32_flag) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* px = x + r * n;
    float* py = y + r * n;
    // optional fused producers: v = x * scale[0] (a Mul by a scalar) and v += mask[row / rows_per_mask][k] (an Add
    // of a mask that broadcasts over heads and query rows), each rounded as the separate nodes would
    const float sc = scale ? scale[0] : 1.f;
    const float* pm = mask ? mask + (r / rows_per_mask) * n : nullptr;
    auto value = [&](int64_t k) {
      float v = px[k];
      if (scale) v = __fmul_rn(v, sc);
      if (pm) v = __fadd_rn(v, pm[k]);
      return v;
    };
    float mx = -INFINITY;
    for (int64_t k = lane; k < n; k += 32) mx = fmaxf(mx, value(k));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int64_t k = lane; k < n; k += 32) {
      const float e = expf(__fsub_rn(value(k), mx));
      py[k] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = __frcp_rn(sum);
    for (int64_t k = lane; k < n; k += 32) {
      const float v = __fmul_rn(py[k], inv);
      py[k] = round_tf32_flag ? round_tf32(v) : v;
    }
  }
}

// The same softmax for rows of 128 * NV4 lanes: a lane keeps its 4 * NV4 values in registers between the three
// phases, so the row is read once and written once, in 16-byte pieces.
template <int NV4>
__global__ void softmax_rows_reg_kernel(const float4* __restrict__ x, float4* __restrict__ y, int64_t rows, const float* __restrict__ scale,
                                        const float4* __restrict__ mask, int64_t rows_per_mask, int round_tf32_flag) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float sc = scale ? scale[0] : 1.f;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float4* px = x + r * (32 * NV4);
    const float4* pm = mask ? mask + (r / rows_per_mask) * (32 * NV4) : nullptr;
    float v[4 * NV4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < NV4; ++j) {
      const float4 t = px[32 * j + lane];
      v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
      if (scale) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[4 * j + e] = __fmul_rn(v[4 * j + e], sc);
      }
      if (pm) {
        const float4 m = __ldg(pm + 32 * j + lane);
        v[4 * j] = __fadd_rn(v[4 * j], m.x), v[4 * j + 1] = __fadd_rn(v[4 * j + 1], m.y), v[4 * j + 2] = __fadd_rn(v[4 * j + 2], m.z),
               v[4 * j + 3] = __fadd_rn(v[4 * j + 3], m.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) mx = fmaxf(mx, v[4 * j + e]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 4 * NV4; ++k) {
      v[k] = expf(__fsub_rn(v[k], mx));
      sum += v[k];
    }
    const float inv = __frcp_rn(warp_sum(sum));
#pragma unroll
    for (int j = 0; j < NV4; ++j) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = __fmul_rn(v[4 * j + e], inv);
        if (round_tf32_flag) o[e] = round_tf32(o[e]);
      }
      y[r * (32 * NV4) + 32 * j + lane] = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
}

// LayerNormalization for rows of 128 * NV4 lanes, the row kept in registers (read once, in 16-byte pieces).
template <int NV4>
__global__ void layer_norm_rows_reg_kernel(const float4* __restrict__ x, const float4* __restrict__ x2, float4* __restrict__ y, int64_t rows,
                                           const float4* __restrict__ scale, const float4* __restrict__ bias, float eps, uint32_t* minmax_keys) {
  const int lane = threadIdx.x & 31;
  const float n = (float)(128 * NV4);
  float mn = INFINITY, mx = -INFINITY;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float4* px = x + r * (32 * NV4);
    float v[4 * NV4];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NV4; ++j) {
      float4 t = px[32 * j + lane];
      if (x2) {  // the Add in front of the normalisation: one rounded sum per lane, as the separate node gives
        const float4 u = x2[r * (32 * NV4) + 32 * j + lane];
        t = make_float4(__fadd_rn(t.x, u.x), __fadd_rn(t.y, u.y), __fadd_rn(t.z, u.z), __fadd_rn(t.w, u.w));
      }
      v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
      sum += (t.x + t.y) + (t.z + t.w);
    }
    const float mean = __fdiv_rn(warp_sum(sum), n);
    float vs = 0.f;
#pragma unroll
    for (int k = 0; k < 4 * NV4; ++k) {
      v[k] = __fsub_rn(v[k], mean);
      vs += __fmul_rn(v[k], v[k]);
    }
    const float var = __fdiv_rn(warp_sum(vs), n);
    const float inv_std = __frcp_rn(__fsqrt_rn(__fadd_rn(var, eps)));
#pragma unroll
    for (int j = 0; j < NV4; ++j) {
      const float4 g = __ldg(scale + 32 * j + lane);
      float o[4] = {__fmul_rn(__fmul_rn(v[4 * j], inv_std), g.x), __fmul_rn(__fmul_rn(v[4 * j + 1], inv_std), g.y),
                    __fmul_rn(__fmul_rn(v[4 * j + 2], inv_std), g.z), __fmul_rn(__fmul_rn(v[4 * j + 3], inv_std), g.w)};
      if (bias) {
        const float4 b = __ldg(bias + 32 * j + lane);
        o[0] = __fadd_rn(o[0], b.x), o[1] = __fadd_rn(o[1], b.y), o[2] = __fadd_rn(o[2], b.z), o[3] = __fadd_rn(o[3], b.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mn = fminf(mn, o[e]);
        mx = fmaxf(mx, o[e]);
      }
      y[r * (32 * NV4) + 32 * j + lane] = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
  if (minmax_keys) {  // uniform across the grid; one pair of atomics per block
    for (int off = 16; off > 0; off >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    __shared__ float smn[kThreads / 32], smx[kThreads / 32];
    const int warp = threadIdx.x >> 5;
    if (lane == 0) {
      smn[warp] = mn;
      smx[warp] = mx;
    }
    __syncthreads();
    if (warp == 0) {
      mn = lane < kThreads / 32 ? smn[lane] : INFINITY;
      mx = lane < kThreads / 32 ? smx[lane] : -INFINITY;
      for (int off = 4; off > 0; off >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      }
      if (lane == 0) {
        if (mn != INFINITY) atomicMin(&minmax_keys[0], float_key(mn));
        if (mx != -INFINITY) atomicMax(&minmax_keys[1], float_key(mx));
      }
    }
  }
}

// LayerNormalization over the last axis, one warp per row (nn/normalization.rs layer_norm_into):
// mean = sum / n, var = sum((x - mean)^2) / n, inv_std = 1 / sqrt(var + eps), (x - mean) * inv_std * scale [+ bias].
__global__ void layer_norm_rows_kernel(const float* __restrict__ x, const float* __restrict__ x2, float* __restrict__ y, int64_t rows, int64_t n,
                                       const float* __restrict__ scale, const float* __restrict__ bias, float eps, uint32_t* minmax_keys) {
  const int lane = threadIdx.x & 31;
  float mn = INFINITY, mx = -INFINITY;  // extrema of what this thread writes (for a DynamicQuantizeLinear reader)
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* px = x + r * n;
    const float* px2 = x2 ? x2 + r * n : nullptr;
    auto at = [&](int64_t k) { return px2 ? __fadd_rn(px[k], px2[k]) : px[k]; };  // the Add in front of the normalisation
    float* py = y + r * n;
    float sum = 0.f;
    for (int64_t k = lane; k < n; k += 32) sum += at(k);
    const float mean = __fdiv_rn(warp_sum(sum), (float)n);
    float vs = 0.f;
    for (int64_t k = lane; k < n; k += 32) {
      const float d = __fsub_rn(at(k), mean);
      vs += __fmul_rn(d, d);
    }
    const float var = __fdiv_rn(warp_sum(vs), (float)n);
    const float inv_std = __frcp_rn(__fsqrt_rn(__fadd_rn(var, eps)));
    for (int64_t k = lane; k < n; k += 32) {
      float v = __fmul_rn(__fmul_rn(__fsub_rn(at(k), mean), inv_std), scale[k]);
      if (bias) v = __fadd_rn(v, bias[k]);
      py[k] = v;
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  if (minmax_keys) {  // uniform across the grid
    for (int off = 16; off > 0; off >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    __shared__ float smn[kThreads / 32], smx[kThreads / 32];
    const int warp = threadIdx.x >> 5;
    if (lane == 0) {
      smn[warp] = mn;
      smx[warp] = mx;
    }
    __syncthreads();
    if (warp == 0) {
      mn = lane < kThreads / 32 ? smn[lane] : INFINITY;
      mx = lane < kThreads / 32 ? smx[lane] : -INFINITY;
      for (int off = 4; off > 0; off >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      }
      if (lane == 0) {
        if (mn != INFINITY) atomicMin(&minmax_keys[0], float_key(mn));
        if (mx != -INFINITY) atomicMax(&minmax_keys[1], float_key(mx));
      }
    }
  }
}

}  // namespace

// =========================================================================================
void convert(const TensorRef& src, const TensorRef& dst, cudaStream_t s) {
  int64_t total = dst.d.numel();
  if (total == 0) return;
  const Dims4& d = dst.d;
  // Coalesced tile transpose for the two hot cases at the graph edges.
  if (src.layout != dst.layout && d.C > 1 && d.H * d.W > 1 && d.N <= 65535) {
    int64_t A, B;  // src viewed [N, A, B] -> dst [N, B, A]
    if (src.layout == Layout::PLAIN) {
      A = d.C;
      B = d.H * d.W;
    } else {
      A = d.H * d.W;
      B = d.C;
    }
    dim3 block(32, 8), grid((unsigned)ceil_div(B, 32), (unsigned)ceil_div(A, 32), (unsigned)d.N);
    if (grid.y <= 65535) {
      if (src.dt == DT::F32 && dst.dt == DT::F32) {
        transpose_tiles<float, float><<<grid, block, 0, s>>>((const float*)src.ptr, (float*)dst.ptr, A, B);
        return;
      }
      if (src.dt == DT::U8 && dst.dt == DT::F32) {
        transpose_tiles<uint8_t, float><<<grid, block, 0, s>>>((const uint8_t*)src.ptr, (float*)dst.ptr, A, B);
        return;
      }
      if (src.dt == DT::I8 && dst.dt == DT::F32) {
        transpose_tiles<int8_t, float><<<grid, block, 0, s>>>((const int8_t*)src.ptr, (float*)dst.ptr, A, B);
        return;
      }
    }
  }
  convert_kernel<<<grid_for(total), kThreads, 0, s>>>(src.ptr, src.dt, src.layout, dst.ptr, dst.dt, dst.layout, d, total);
}

// Eight lanes per thread: two 16-byte loads, one 16-byte store; the tail runs lane by lane.
__global__ void f32_to_half_kernel(const float* __restrict__ src, void* __restrict__ dst, bool bf16, int64_t n8, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * i), b = __ldg(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    uint4 o;
    if (bf16) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w), p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
      o = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1), *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
    } else {
      __half2 p0 = __floats2half2_rn(a.x, a.y), p1 = __floats2half2_rn(a.z, a.w), p2 = __floats2half2_rn(b.x, b.y), p3 = __floats2half2_rn(b.z, b.w);
      o = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1), *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
    }
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
  for (int64_t i = n8 * 8 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) {
    if (bf16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(src[i]);
    else reinterpret_cast<__half*>(dst)[i] = __float2half_rn(src[i]);
  }
}

__global__ void round_to_tf32_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n4, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src) + i);
    reinterpret_cast<float4*>(dst)[i] = make_float4(round_tf32(a.x), round_tf32(a.y), round_tf32(a.z), round_tf32(a.w));
  }
  for (int64_t i = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = round_tf32(src[i]);
}

void round_to_tf32_copy(const float* src, float* dst, int64_t n, cudaStream_t s) {
  if (n == 0) return;
  const int64_t n4 = ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) ? n / 4 : 0;
  round_to_tf32_kernel<<<grid_for(std::max<int64_t>(n4, n - n4 * 4)), kThreads, 0, s>>>(src, dst, n4, n);
}

void convert_f32_to_half(const float* src, void* dst, DT dst_dt, int64_t n, cudaStream_t s) {
  if (n == 0) return;
  if (!(dst_dt == DT::F16 || dst_dt == DT::BF16)) OXB_FAIL("convert_f32_to_half: destination is not a 16-bit float type");
  const int64_t n8 = ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) ? n / 8 : 0;
  f32_to_half_kernel<<<grid_for(std::max<int64_t>(n8, n - n8 * 8)), kThreads, 0, s>>>(src, dst, dst_dt == DT::BF16, n8, n);
}

void residual_requant(const void* a, DT a_dt, const void* b, DT b_dt, void* y, DT y_dt, int64_t n, const ResidualParams& rp, cudaStream_t s) {
  (void)y_dt;
  if (n == 0) return;
  const bool as = a_dt == DT::I8, bs = b_dt == DT::I8;
  int64_t n16 = 0;
  if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 15) == 0) n16 = n / 16;
  if (n16 > 0) {
    if (rp.proven_fast == 2) residual_requant_kernel<2><<<grid_for(n16), kThreads, 0, s>>>((const uint4*)a, as, (const uint4*)b, bs, (uint4*)y, n16, rp);
    else if (rp.proven_fast == 1) residual_requant_kernel<1><<<grid_for(n16), kThreads, 0, s>>>((const uint4*)a, as, (const uint4*)b, bs, (uint4*)y, n16, rp);
    else residual_requant_kernel<0><<<grid_for(n16), kThreads, 0, s>>>((const uint4*)a, as, (const uint4*)b, bs, (uint4*)y, n16, rp);
  }
  if (n16 * 16 < n)
    residual_requant_tail_kernel<<<grid_for(n - n16 * 16), kThreads, 0, s>>>((const uint8_t*)a, as, (const uint8_t*)b, bs, (uint8_t*)y, n16 * 16, n, rp);
}

// Host restatement of both device formulas (IEEE single precision, one rounding per operation,
// fused multiply-add through fmaf), compared over every pair of input bytes.
void residual_requant_prepare(ResidualParams& rp, DT a_dt, DT b_dt) {
  rp.proven_fast = 0;
  rp.y_rcp = 0.f;
  auto sane = [](float v) { return std::isfinite(v) && std::fabs(v) >= 9.5367431640625e-07f && std::fabs(v) <= 1048576.0f; };  // 2^-20 .. 2^20
  if (!sane(rp.a_scale) || !sane(rp.b_scale) || !sane(rp.y_scale)) return;
  if (!(std::fabs(rp.a_zp) <= 255.f && std::fabs(rp.b_zp) <= 255.f && std::fabs(rp.y_zp) <= 255.f)) return;
  const float y_rcp = (float)(1.0 / (double)rp.y_scale);
  const int a_lo = a_dt == DT::I8 ? -128 : 0, b_lo = b_dt == DT::I8 ? -128 : 0;
  const float magic = 12582912.0f;
  const float lo_eff = rp.relu ? std::fmax(rp.lo, rp.y_zp) : rp.lo;
  bool packed_ok = rp.y_scale > 0.f && std::fabs(rp.lo) <= 32000.f && std::fabs(rp.hi) <= 32000.f;
  for (int ia = a_lo; ia < a_lo + 256; ++ia) {
    volatile float va = ((float)ia - rp.a_zp) * rp.a_scale;
    for (int ib = b_lo; ib < b_lo + 256; ++ib) {
      volatile float vb = ((float)ib - rp.b_zp) * rp.b_scale;
      volatile float sum = va + vb;
      if (rp.relu) sum = std::fmax(sum, 0.f);
      // reference: round_ties_even(sum / y_scale) + zero point, clamped
      volatile float quot = sum / rp.y_scale;
      volatile float ref = std::nearbyintf(quot) + rp.y_zp;
      const float want = std::fmin(std::fmax(ref, rp.lo), rp.hi);
      // fast path
      volatile float q0 = sum * y_rcp;
      volatile float rem = std::fmaf(-q0, rp.y_scale, sum);
      volatile float q = std::fmaf(rem, y_rcp, q0);
      volatile float t1 = q + magic;
      volatile float t = t1 + rp.y_zp;
      const float got = std::fmin(std::fmax(t, magic + rp.lo), magic + rp.hi) - magic;
      if (!(got == want)) return;
      if (packed_ok) {
        // the pairwise form: no ReLU on the sum, the same quotient, the low half-word of t clamped as an int16
        volatile float sum2 = va + vb;
        volatile float p0 = sum2 * y_rcp;
        volatile float prem = std::fmaf(p0, -rp.y_scale, sum2);
        volatile float pq = std::fmaf(prem, y_rcp, p0);
        volatile float pt1 = pq + magic;
        volatile float pt = pt1 + rp.y_zp;
        const float ti = pt - magic;  // exact: pt is an integer of the binade when it is in range
        if (!(pt >= 8388608.0f && pt < 16777216.0f) || std::fabs(ti) > 32000.f) packed_ok = false;
        else if (!(std::fmin(std::fmax(ti, lo_eff), rp.hi) == want)) packed_ok = false;
      }
    }
  }
  rp.y_rcp = y_rcp;
  rp.proven_fast = packed_ok ? 2 : 1;
}

void s2d_pack(const TensorRef& src, void* dst, DT dst_dt, int c_pad, int sub, cudaStream_t s) {
  int64_t total4 = src.d.N * (src.d.H / 2) * (src.d.W / 2) * (c_pad / 4);
  if (total4 == 0) return;
  if (!(dst_dt == DT::F32 || dst_dt == DT::U8 || dst_dt == DT::I8)) OXB_FAIL("s2d_pack: unsupported storage type");
  s2d_pack_kernel<<<grid_for(total4), kThreads, 0, s>>>(src.ptr, src.dt, src.layout, src.d, dst, dst_dt, c_pad, sub, total4);
}

void s2d_window_pack(const TensorRef& src, void* dst, DT dst_dt, int pad_left, int wp, int sub, const S2dQuant& q, int pair_top, int rows_phys,
                     cudaStream_t s) {
  const int64_t total = src.d.N * (pair_top >= 0 ? (int64_t)rows_phys + 1 : src.d.H / 2) * wp;
  if (total == 0) return;
  if (!(dst_dt == DT::F32 || dst_dt == DT::U8 || dst_dt == DT::I8) || 4 * src.d.C > 16) OXB_FAIL("s2d_window_pack: unsupported operand");
  if (pair_top >= 0 && dst_dt == DT::F32) OXB_FAIL("s2d_window_pack: row pairs are an 8-bit layout");
  if (q.quantize && src.dt != DT::F32) OXB_FAIL("s2d_window_pack: quantisation needs an f32 source");
  if (src.dt == DT::F32 && src.layout == Layout::PLAIN && src.d.W % 2 == 0 && ((uintptr_t)src.ptr & 7) == 0 && src.d.C >= 1 && src.d.C <= 4) {
    const bool safe = q.quantize && q.scale >= 7.8886090522101181e-31f && q.scale <= 1.2676506002282294e+30f;
    const float rcp = safe ? 1.0f / q.scale : 0.f;
    const int g = grid_for(total);
    const float* x = (const float*)src.ptr;
    switch ((int)src.d.C) {
      case 1: s2d_window_pack_nchw_f32_kernel<1><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, q, rcp, safe, total, pair_top, rows_phys); break;
      case 2: s2d_window_pack_nchw_f32_kernel<2><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, q, rcp, safe, total, pair_top, rows_phys); break;
      case 3: s2d_window_pack_nchw_f32_kernel<3><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, q, rcp, safe, total, pair_top, rows_phys); break;
      default: s2d_window_pack_nchw_f32_kernel<4><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, q, rcp, safe, total, pair_top, rows_phys); break;
    }
    return;
  }
  if ((src.dt == DT::U8 || src.dt == DT::I8) && (dst_dt == DT::U8 || dst_dt == DT::I8) && src.layout == Layout::PLAIN && src.d.W % 2 == 0 &&
      ((uintptr_t)src.ptr & 1) == 0 && src.d.C >= 1 && src.d.C <= 4 && !q.quantize) {
    const int g = grid_for(total);
    const uint8_t* x = (const uint8_t*)src.ptr;
#define OXB_Q8_PACK(CC)                                                                                                                          \
  if (src.dt == DT::I8) s2d_window_pack_nchw_q8_kernel<CC, true><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, total, pair_top, rows_phys); \
  else s2d_window_pack_nchw_q8_kernel<CC, false><<<g, kThreads, 0, s>>>(x, src.d, dst, dst_dt, pad_left, wp, sub, total, pair_top, rows_phys);
    switch ((int)src.d.C) {
      case 1: OXB_Q8_PACK(1) break;
      case 2: OXB_Q8_PACK(2) break;
      case 3: OXB_Q8_PACK(3) break;
      default: OXB_Q8_PACK(4) break;
    }
#undef OXB_Q8_PACK
    return;
  }
  s2d_window_pack_kernel<<<grid_for(total), kThreads, 0, s>>>(src.ptr, src.dt, src.layout, src.d, dst, dst_dt, pad_left, wp, sub, q, total, pair_top, rows_phys);
}

void window_pack_f32(const TensorRef& src, void* dst, int pad_left, int wp, cudaStream_t s) {
  const int64_t total = src.d.N * src.d.H * wp;
  if (total == 0) return;
  if (src.dt != DT::F32 || src.d.C > 4) OXB_FAIL("window_pack_f32: unsupported operand");
  window_pack_f32_kernel<<<grid_for(total), kThreads, 0, s>>>((const float*)src.ptr, src.layout, src.d, (float4*)dst, pad_left, wp, total);
}

void quantize_linear(const TensorRef& x, const TensorRef& y, const float* scale, int64_t n_scale, const float* zp, int64_t n_zp, float lo,
                     float hi, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  quantize_kernel<<<grid_for(total), kThreads, 0, s>>>(x.ptr, x.dt, x.layout, y.ptr, y.dt, y.layout, y.d, scale, n_scale, zp, n_zp, lo, hi,
                                                       total);
}

bool quantize_linear_scalar_ok(const TensorRef& x, const TensorRef& y) {
  int64_t total = y.d.numel();
  bool same_order = x.layout == y.layout || (y.d.C == 1) || (y.d.H * y.d.W == 1);
  return x.dt == DT::F32 && (y.dt == DT::U8 || y.dt == DT::I8) && same_order && total > 0 && total % 16 == 0 &&
         ((uintptr_t)x.ptr % 16 == 0) && ((uintptr_t)y.ptr % 16 == 0);
}

// Host-known per-tensor parameters: the vectorised kernel.
void quantize_linear_scalar(const TensorRef& x, const TensorRef& y, float scale, float zp, float lo, float hi, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (quantize_linear_scalar_ok(x, y)) {
    quantize_vec16_kernel<<<grid_for(total / 16), kThreads, 0, s>>>((const float4*)x.ptr, (uint4*)y.ptr, scale, zp, lo, hi, total / 16);
    return;
  }
  OXB_FAIL("quantize_linear_scalar: no vector path for this operand");
}

void dequantize_linear(const TensorRef& x, const TensorRef& y, const float* scale, int64_t n_scale, const float* zp, int64_t n_zp,
                       cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  const bool same_order = x.layout == y.layout || y.d.C == 1 || y.d.H * y.d.W == 1;
  if ((x.dt == DT::U8 || x.dt == DT::I8) && n_scale == 1 && n_zp <= 1 && same_order && total % 4 == 0 && ((uintptr_t)x.ptr & 3) == 0 &&
      ((uintptr_t)y.ptr & 15) == 0) {
    dequantize_vec4_kernel<<<grid_for(total / 4), kThreads, 0, s>>>((const uint32_t*)x.ptr, x.dt == DT::I8, (float4*)y.ptr, scale, zp, total / 4);
    return;
  }
  dequantize_kernel<<<grid_for(total), kThreads, 0, s>>>(x.ptr, x.dt, x.layout, y.ptr, y.layout, y.d, scale, n_scale, zp, n_zp, total);
}

void dynamic_quantize_linear(const TensorRef& x, const TensorRef& y, float* params, float* scratch, cudaStream_t s, bool have_minmax) {
  // `scratch` holds {min key, max key, arrival counter}, set to {0xffffffff, 0, 0} when it was allocated
  // (dynamic_quantize_scratch_init) and put back to that by the last block of every apply pass
  int64_t n = x.d.numel();
  uint32_t* keys = (uint32_t*)scratch;
  if ((((uintptr_t)x.ptr) & 15) != 0 || (((uintptr_t)y.ptr) & 3) != 0) {
    // operands that are not aligned for 16-byte loads / 4-byte stores: the same arithmetic, one lane per access
    if (!have_minmax) minmax_kernel<<<grid_for(n), kThreads, 0, s>>>((const float*)x.ptr, n, keys, 0);
    dynq_apply_fused_kernel<<<grid_for(n), kThreads, 0, s>>>((const float*)x.ptr, (uint8_t*)y.ptr, keys, params, n, 0);
    return;
  }
  const int64_t cap = 148 * 8;
  const int64_t b_mm = std::min<int64_t>(cap, std::max<int64_t>(1, (n / 4 + kThreads * 4 - 1) / (kThreads * 4)));
  const int64_t b_ap = std::min<int64_t>(cap, std::max<int64_t>(1, (n / 4 + (kThreads / 32) * 128 - 1) / ((kThreads / 32) * 128)));
  if (!have_minmax) minmax_wide_kernel<<<(int)b_mm, kThreads, 0, s>>>((const float*)x.ptr, n, keys);
  dynq_apply_wide_kernel<<<(int)b_ap, kThreads, 0, s>>>((const float*)x.ptr, (uint8_t*)y.ptr, keys, params, n);
}

void dynamic_quantize_scratch_init(float* scratch) {
  const uint32_t init[3] = {0xffffffffu, 0u, 0u};
  OXB_CUDA(cudaMemcpy(scratch, init, sizeof init, cudaMemcpyHostToDevice));
}

void binary(const TensorRef& a, const TensorRef& b, const TensorRef& out, int op, int relu_after, int round_tf32_flag, cudaStream_t s) {
  int64_t total = out.d.numel();
  if (total == 0) return;
  bool same = a.d.numel() == total && b.d.numel() == total && a.layout == out.layout && b.layout == out.layout && a.dt == DT::F32 &&
              b.dt == DT::F32 && out.dt == DT::F32 && total % 4 == 0;
  if (same) {
    binary_vec4_kernel<<<grid_for(total / 4), kThreads, 0, s>>>((const float4*)a.ptr, (const float4*)b.ptr, (float4*)out.ptr, op, relu_after,
                                                               round_tf32_flag, total / 4);
    return;
  }
  if (a.d.numel() == total && a.layout == Layout::PLAIN && b.layout == Layout::PLAIN && out.layout == Layout::PLAIN && a.dt == DT::F32 && b.dt == DT::F32 &&
      out.dt == DT::F32 && total % 4 == 0 && total / 4 < (int64_t)1 << 31 && (((uintptr_t)a.ptr | (uintptr_t)b.ptr | (uintptr_t)out.ptr) & 15) == 0) {
    const int64_t od[4] = {out.d.N, out.d.C, out.d.H, out.d.W}, bd[4] = {b.d.N, b.d.C, b.d.H, b.d.W};
    int k0 = 0;
    while (k0 < 4 && bd[k0] == 1) ++k0;
    bool suffix = k0 > 0 && k0 < 4;
    int64_t nb = 1;
    for (int j = k0; j < 4; ++j) {
      suffix = suffix && bd[j] == od[j];
      nb *= bd[j];
    }
    if (suffix && nb % 4 == 0) {
      binary_suffix_vec4_kernel<<<grid_for(total / 4), kThreads, 0, s>>>((const float4*)a.ptr, (const float4*)b.ptr, (float4*)out.ptr, op, relu_after,
                                                                         round_tf32_flag, (uint32_t)(total / 4), (uint32_t)(nb / 4));
      return;
    }
  }
  binary_kernel<<<grid_for(total), kThreads, 0, s>>>(a.ptr, a.dt, a.layout, a.d, b.ptr, b.dt, b.layout, b.d, out.ptr, out.dt, out.layout,
                                                     out.d, op, relu_after, round_tf32_flag, total);
}

void unary(const TensorRef& x, const TensorRef& y, int op, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  unary_kernel<<<grid_for(total), kThreads, 0, s>>>(x.ptr, x.dt, y.ptr, y.dt, op, total);
}

void prelu(const TensorRef& x, const TensorRef& y, const float* slope, int64_t n_slope, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  prelu_kernel<<<grid_for(total), kThreads, 0, s>>>((const float*)x.ptr, x.layout, (float*)y.ptr, x.d, slope, n_slope, total);
}

void max_pool(const TensorRef& x, const TensorRef& y, const PoolShape& ps, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  const int64_t per = x.dt == DT::F32 ? 4 : 16;
  if (x.d.C % per == 0 && (((uintptr_t)x.ptr | (uintptr_t)y.ptr) & 15) == 0 && (x.dt == DT::F32 || x.dt == DT::U8 || x.dt == DT::I8)) {
    const int64_t cvec = x.d.C / per, tv = total / per;
    const int gv = grid_for(tv);
    if (ps.kh == 3 && ps.kw == 3 && ps.sh == 2 && ps.sw == 2 && ps.dh == 1 && ps.dw == 1 && ps.pt == 1 && ps.pl == 1 && tv < 0x7fffffffLL &&
        x.d.numel() / per < 0x7fffffffLL) {
      const int H = (int)x.d.H, W = (int)x.d.W, cv = (int)cvec, n = (int)tv;
      if (x.dt == DT::F32) max_pool_3x3s2_kernel<0><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, H, W, ps.P, ps.Q, cv, n);
      else if (x.dt == DT::U8) max_pool_3x3s2_kernel<1><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, H, W, ps.P, ps.Q, cv, n);
      else max_pool_3x3s2_kernel<2><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, H, W, ps.P, ps.Q, cv, n);
      return;
    }
    if (x.dt == DT::F32) max_pool_nhwc_vec_kernel<0><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, x.d, ps, cvec, tv);
    else if (x.dt == DT::U8) max_pool_nhwc_vec_kernel<1><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, x.d, ps, cvec, tv);
    else max_pool_nhwc_vec_kernel<2><<<gv, kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, x.d, ps, cvec, tv);
    return;
  }
  int g = grid_for(total);
  if (x.dt == DT::F32) max_pool_nhwc_kernel<float><<<g, kThreads, 0, s>>>((const float*)x.ptr, (float*)y.ptr, x.d, ps, total, -INFINITY);
  else if (x.dt == DT::U8) max_pool_nhwc_kernel<uint8_t><<<g, kThreads, 0, s>>>((const uint8_t*)x.ptr, (uint8_t*)y.ptr, x.d, ps, total, 0);
  else if (x.dt == DT::I8) max_pool_nhwc_kernel<int8_t><<<g, kThreads, 0, s>>>((const int8_t*)x.ptr, (int8_t*)y.ptr, x.d, ps, total, -128);
  else OXB_FAIL("max_pool: unsupported storage type");
}

void global_avg_pool_dequant(const TensorRef& x, const TensorRef& y, float scale, float zp, int round_tf32_flag, cudaStream_t s) {
  if (!(x.dt == DT::U8 || x.dt == DT::I8) || x.d.C % 4 != 0 || ((uintptr_t)x.ptr & 3) != 0 || ((uintptr_t)y.ptr & 15) != 0)
    OXB_FAIL("global_avg_pool_dequant: unsupported operand");
  const int64_t total4 = x.d.N * x.d.C / 4;
  if (total4 == 0) return;
  global_avg_pool_nhwc_q_kernel<<<grid_for(total4, 128), 128, 0, s>>>((const uint32_t*)x.ptr, x.dt == DT::I8, scale, zp, (float4*)y.ptr, x.d, round_tf32_flag);
}

void global_avg_pool(const TensorRef& x, const TensorRef& y, int round_tf32_flag, cudaStream_t s) {
  int64_t total = x.d.N * x.d.C;
  if (total == 0) return;
  global_avg_pool_nhwc_kernel<<<grid_for(total, 128), 128, 0, s>>>((const float*)x.ptr, (float*)y.ptr, x.d, round_tf32_flag);
}

void instance_norm(const TensorRef& x, const TensorRef& y, float eps, const float* scale_nc, const float* shift_nc, int relu, int round_tf32_flag,
                   cudaStream_t s) {
  int64_t cgroups = (x.d.C + 31) / 32;
  int64_t blocks = x.d.N * cgroups;
  if (blocks == 0) return;
  const int64_t hw = x.d.H * x.d.W;
  const size_t slab = (size_t)hw * 32 * sizeof(float);
  if (hw >= 256 && slab <= 200 * 1024) {
    // the opt-in for more than 48 KB of dynamic shared memory is a per-device property of the kernel
    static std::mutex mu;
    static size_t have[64] = {};
    int dev = 0;
    OXB_CUDA(cudaGetDevice(&dev));
    {
      std::lock_guard<std::mutex> lock(mu);
      size_t& h = have[dev >= 0 && dev < 64 ? dev : 0];
      if (slab > h) {
        OXB_CUDA(cudaFuncSetAttribute(instance_norm_nhwc_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slab));
        h = slab;
      }
    }
    instance_norm_nhwc_smem_kernel<<<(unsigned)blocks, 1024, slab, s>>>((const float*)x.ptr, (float*)y.ptr, x.d, eps, scale_nc, shift_nc, relu,
                                                                        round_tf32_flag);
    return;
  }
  instance_norm_nhwc_kernel<<<(unsigned)blocks, 256, 0, s>>>((const float*)x.ptr, (float*)y.ptr, x.d, eps, scale_nc, shift_nc, relu, round_tf32_flag);
}

void resize(const TensorRef& x, const TensorRef& y, int mode, int coord, int nearest_rule, float scale_h, float scale_w, int round_tf32_flag,
            cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  if (y.d.C % 4 == 0 && ((uintptr_t)x.ptr & 15) == 0 && ((uintptr_t)y.ptr & 15) == 0) {
    if (total / 4 + (int64_t)148 * 64 * kThreads < (int64_t)1 << 31)
      resize_nhwc_vec4_kernel<uint32_t><<<grid_for(total / 4), kThreads, 0, s>>>((const float4*)x.ptr, (float4*)y.ptr, x.d, y.d, mode, coord, nearest_rule,
                                                                                scale_h, scale_w, total / 4, round_tf32_flag);
    else
      resize_nhwc_vec4_kernel<int64_t><<<grid_for(total / 4), kThreads, 0, s>>>((const float4*)x.ptr, (float4*)y.ptr, x.d, y.d, mode, coord, nearest_rule,
                                                                               scale_h, scale_w, total / 4, round_tf32_flag);
    return;
  }
  resize_nhwc_kernel<<<grid_for(total), kThreads, 0, s>>>((const float*)x.ptr, (float*)y.ptr, x.d, y.d, mode, coord, nearest_rule, scale_h,
                                                          scale_w, total, round_tf32_flag);
}

void pad(const TensorRef& x, const TensorRef& y, int mode, float value, int pn, int pc, int ph, int pw, cudaStream_t s) {
  int64_t total = y.d.numel();
  if (total == 0) return;
  const size_t es = x.dt == DT::F32 || x.dt == DT::I32 ? 4 : (x.dt == DT::I16 ? 2 : 1);
  if (x.layout == Layout::NHWC && pn == 0 && pc == 0 && (x.d.C * es) % 16 == 0 && ((uintptr_t)x.ptr & 15) == 0 && ((uintptr_t)y.ptr & 15) == 0) {
    // the fill value in the tensor's storage type, replicated over 16 bytes
    uint32_t word;  // rounded to nearest even and saturated like store_from_f32
    auto sat = [&](float lo, float hi) { return (int32_t)std::nearbyint(std::fmin(std::fmax(value, lo), hi)); };
    if (x.dt == DT::F32) {
      std::memcpy(&word, &value, 4);
    } else if (x.dt == DT::I32) {
      const int32_t iv = (int32_t)std::nearbyint(std::fmin(std::fmax(value, -2147483648.0f), 2147483520.0f));
      std::memcpy(&word, &iv, 4);
    } else if (x.dt == DT::I16) {
      const uint16_t hv = (uint16_t)(int16_t)sat(-32768.f, 32767.f);
      word = (uint32_t)hv | ((uint32_t)hv << 16);
    } else {
      const uint8_t bv = x.dt == DT::U8 ? (uint8_t)sat(0.f, 255.f) : (uint8_t)(int8_t)sat(-128.f, 127.f);
      word = bv * 0x01010101u;
    }
    const int64_t vpp = (int64_t)(x.d.C * es / 16);
    const int64_t total_v = y.d.N * y.d.H * y.d.W * vpp;
    if (total_v + (int64_t)148 * 64 * kThreads < (int64_t)1 << 31)
      pad_nhwc_vec_kernel<uint32_t><<<grid_for(total_v), kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, x.d, y.d, vpp, mode,
                                                                          make_uint4(word, word, word, word), ph, pw, total_v);
    else
      pad_nhwc_vec_kernel<int64_t><<<grid_for(total_v), kThreads, 0, s>>>((const uint4*)x.ptr, (uint4*)y.ptr, x.d, y.d, vpp, mode,
                                                                         make_uint4(word, word, word, word), ph, pw, total_v);
    return;
  }
  pad_kernel<<<grid_for(total), kThreads, 0, s>>>(x.ptr, y.ptr, x.dt, x.layout, x.d, y.d, mode, value, pn, pc, ph, pw, total);
}

void slice_rows(const void* x, void* y, DT dt, const Dims4& xd, const Dims4& yd, const Dims4& start, cudaStream_t s) {
  const int64_t total = yd.numel();
  if (total == 0) return;
  const int es = dt == DT::F32 || dt == DT::I32 ? 4 : (dt == DT::I16 ? 2 : 1);
  slice_kernel<<<grid_for(total), kThreads, 0, s>>>(x, y, es, xd, yd, start, total);
}

void gather_rows(const float* table, const float* idx, float* out, int64_t n_idx, int64_t rows, int64_t inner, int* err, cudaStream_t s) {
  if (n_idx * inner == 0) return;
  gather_rows_kernel<<<grid_for(n_idx * inner), kThreads, 0, s>>>(table, idx, out, n_idx, rows, inner, err);
}

void transpose_perm(const void* x, void* y, const Dims4& yd, const Dims4& xstride, cudaStream_t s) {
  const int64_t total = yd.numel();
  if (total == 0) return;
  if (xstride.W == 1 && yd.W % 4 == 0 && xstride.N % 4 == 0 && xstride.C % 4 == 0 && xstride.H % 4 == 0 && total < (int64_t)1 << 31 &&
      ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0) {
    const uint32_t total4 = (uint32_t)(total / 4);
    transpose_perm_vec4_kernel<<<grid_for(total4), kThreads, 0, s>>>((const uint4*)x, (uint4*)y, (uint32_t)yd.C, (uint32_t)yd.H, (uint32_t)(yd.W / 4),
                                                                     (uint32_t)(xstride.N / 4), (uint32_t)(xstride.C / 4), (uint32_t)(xstride.H / 4), total4);
    return;
  }
  if (xstride.H == 1 && xstride.W != 1 && yd.H % 4 == 0 && yd.W % 4 == 0 && yd.H >= 8 && yd.W >= 32 && xstride.W % 4 == 0 && xstride.N % 4 == 0 &&
      xstride.C % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0) {
    const int64_t blocks = yd.N * yd.C * ((yd.H + 31) / 32) * ((yd.W + 127) / 128);
    transpose_tiled_vec4_kernel<<<(unsigned)std::min<int64_t>(blocks, 148 * 64), 256, 0, s>>>((const float*)x, (float*)y, yd, xstride, blocks);
    return;
  }
  if (xstride.H == 1 && xstride.W != 1 && yd.H >= 8 && yd.W >= 8) {
    const int64_t blocks = yd.N * yd.C * ((yd.H + 31) / 32) * ((yd.W + 31) / 32);
    transpose_tiled_kernel<<<(unsigned)std::min<int64_t>(blocks, 148 * 64), 256, 0, s>>>((const uint32_t*)x, (uint32_t*)y, yd, xstride, blocks);
    return;
  }
  transpose_perm_kernel<<<grid_for(total), kThreads, 0, s>>>((const uint32_t*)x, (uint32_t*)y, yd, xstride, total);
}

void softmax_rows(const float* x, float* y, int64_t rows, int64_t n, const float* scale, const float* mask, int64_t rows_per_mask, int round_tf32_flag,
                  cudaStream_t s) {
  if (rows * n == 0) return;
  const int64_t rpm = rows_per_mask > 0 ? rows_per_mask : 1;
  if (n % 128 == 0 && n <= 512 && n != 384 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)mask) & 15) == 0) {
    const int g = grid_for(rows * 32);
    const float4 *x4 = (const float4*)x, *m4 = (const float4*)mask;
    if (n == 128) softmax_rows_reg_kernel<1><<<g, kThreads, 0, s>>>(x4, (float4*)y, rows, scale, m4, rpm, round_tf32_flag);
    else if (n == 256) softmax_rows_reg_kernel<2><<<g, kThreads, 0, s>>>(x4, (float4*)y, rows, scale, m4, rpm, round_tf32_flag);
    else softmax_rows_reg_kernel<4><<<g, kThreads, 0, s>>>(x4, (float4*)y, rows, scale, m4, rpm, round_tf32_flag);
    return;
  }
  softmax_rows_kernel<<<grid_for(rows * 32), kThreads, 0, s>>>(x, y, rows, n, scale, mask, rpm, round_tf32_flag);
}

void layer_norm_rows(const float* x, float* y, int64_t rows, int64_t n, const float* scale, const float* bias, float eps, cudaStream_t s,
                     unsigned int* minmax_keys, const float* x2) {
  if (rows * n == 0) return;
  if (n % 256 == 0 && n <= 1024 && (((uintptr_t)x | (uintptr_t)x2 | (uintptr_t)y | (uintptr_t)scale | (uintptr_t)bias) & 15) == 0) {
    const int g = grid_for(rows * 32);
    const float4 *x4 = (const float4*)x, *x24 = (const float4*)x2, *s4 = (const float4*)scale, *b4 = (const float4*)bias;
    if (n == 256) layer_norm_rows_reg_kernel<2><<<g, kThreads, 0, s>>>(x4, x24, (float4*)y, rows, s4, b4, eps, minmax_keys);
    else if (n == 512) layer_norm_rows_reg_kernel<4><<<g, kThreads, 0, s>>>(x4, x24, (float4*)y, rows, s4, b4, eps, minmax_keys);
    else if (n == 768) layer_norm_rows_reg_kernel<6><<<g, kThreads, 0, s>>>(x4, x24, (float4*)y, rows, s4, b4, eps, minmax_keys);
    else layer_norm_rows_reg_kernel<8><<<g, kThreads, 0, s>>>(x4, x24, (float4*)y, rows, s4, b4, eps, minmax_keys);
    return;
  }
  layer_norm_rows_kernel<<<grid_for(rows * 32), kThreads, 0, s>>>(x, x2, y, rows, n, scale, bias, eps, minmax_keys);
}

void concat_into(const TensorRef& x, const TensorRef& y, int axis, int64_t offset, cudaStream_t s) {
  int64_t total = x.d.numel();
  if (total == 0) return;
  concat_kernel<<<grid_for(total), kThreads, 0, s>>>(x.ptr, y.ptr, x.dt, x.layout, x.d, y.d, axis, offset, total);
}

// =========================================================================================
// DynamicQuantizeLinear for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: inside a real-time
// frame loop whose memory was carved up at start-up, inside another runtime's arena that owns
// every byte of the device, or in a sandboxed plug-in that is simply not allowed to call the
// allocator.  The ordinary path keeps its min/max reduction words in memory it allocates; this
// variant keeps them in a small array that is part of the library image instead, so it calls no
// cudaMalloc, no cudaFree and no allocating library routine.  Every GPU that loads the library
// carries the array (256 bytes) until the process exits.
//
// The array's name is only a host-side handle in host code: the kernels need its device address,
// which is looked up once per device with cudaGetSymbolAddress while that device is current.
// That look-up happens inside the first call made for a device, so the first call should be made
// before any stream capture begins.  All calls share the one array and it keeps whatever the
// previous call left there: each call re-initialises the two reduction words on its stream before
// using them, and two calls that overlap on the same GPU (different streams, or different host
// threads) race on it and must be serialised by the caller.
namespace {

constexpr unsigned long long kNoAllocMaxElems = 1ull << 28;  // 268,435,456 lanes (1 GiB of f32 input)
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned int g_noalloc_scratch[64];

std::mutex g_noalloc_mutex;
unsigned int* g_noalloc_scratch_addr[kNoAllocMaxDevices] = {};

}  // namespace
}  // namespace k
}  // namespace oxb

extern "C" int oxb200_dynamic_quantize_linear_noalloc(int device_ordinal, const float* x_device, uint64_t n, uint8_t* y_device,
                                                       float* scale_zp_device, void* cuda_stream) {
  using namespace oxb;
  using namespace oxb::k;
  auto fail = [](const std::string& m) {
    set_thread_error(m);
    return (int)OXB200_FAILED;
  };
  if (!x_device || !y_device || !scale_zp_device) return fail("dynamic_quantize_linear_noalloc: NULL device pointer");
  if (n == 0) return fail("dynamic_quantize_linear_noalloc: input is empty");
  if (n > kNoAllocMaxElems) {
    char buf[160];
    snprintf(buf, sizeof buf, "dynamic_quantize_linear_noalloc: %llu lanes exceed the maximum of %llu for the allocation-free entry point",
             (unsigned long long)n, kNoAllocMaxElems);
    return fail(buf);
  }
  if (device_ordinal < 0 || device_ordinal >= kNoAllocMaxDevices) return fail("dynamic_quantize_linear_noalloc: device ordinal out of range");
  // the kernels read x in 16-byte pieces and write y in 4-byte words: a sub-buffer at an odd offset would fault on the device
  if (((uintptr_t)x_device & 15) != 0) return fail("dynamic_quantize_linear_noalloc: x_device must be 16-byte aligned");
  if (((uintptr_t)y_device & 3) != 0) return fail("dynamic_quantize_linear_noalloc: y_device must be 4-byte aligned");
  if (((uintptr_t)scale_zp_device & 3) != 0) return fail("dynamic_quantize_linear_noalloc: scale_zp_device must be 4-byte aligned");
  int previous = -1;
  if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
  cudaError_t e = cudaSetDevice(device_ordinal);
  if (e != cudaSuccess) return fail(std::string("dynamic_quantize_linear_noalloc: cudaSetDevice: ") + cudaGetErrorString(e));
  unsigned int* scratch = nullptr;
  {
    // set-up, once per device, with that device current
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_scratch_addr[device_ordinal]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p) {
        if (previous >= 0) cudaSetDevice(previous);
        return fail(std::string("dynamic_quantize_linear_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
      }
      g_noalloc_scratch_addr[device_ordinal] = (unsigned int*)p;
    }
    scratch = g_noalloc_scratch_addr[device_ordinal];
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const int64_t count = (int64_t)n;
  minmax_init_kernel<<<1, 1, 0, s>>>(scratch);  // the shared words start every call from their identity values
  minmax_kernel<<<grid_for(count / 4 + 1), kThreads, 0, s>>>(x_device, count, scratch, 1);
  dynq_params_kernel<<<1, 1, 0, s>>>(scratch, scale_zp_device);
  dynq_apply_kernel<<<grid_for(count / 4 + 1), kThreads, 0, s>>>(x_device, y_device, scale_zp_device, count);
  e = cudaGetLastError();
  if (previous >= 0 && previous != device_ordinal) cudaSetDevice(previous);
  if (e != cudaSuccess) return fail(std::string("dynamic_quantize_linear_noalloc: launch failed: ") + cudaGetErrorString(e));
  return (int)OXB200_OK_DEVICE;
}
