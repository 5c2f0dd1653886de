// Direct CUDA-core contractions (sm_100a).  These kernels take every geometry and every
// zero-point combination the reference's integer_conv / integer_matmul accept (groups,
// dilations, asymmetric pads, per-channel weight zero points, per-row matmul zero points)
// and subtract the zero points element by element with padding taps skipped, exactly like
// oxionnx-ops/src/registry/quant_ops/conv_kernel.rs:205-249.  They are the path for nodes
// the tensor-core kernel is not eligible for; the hot layers go through kernels_umma.cu.
#include "kernels.hpp"

namespace oxb {
namespace k {

namespace {

template <typename T>
__device__ __forceinline__ int32_t as_int(T v) {
  return (int32_t)v;
}
template <>
__device__ __forceinline__ int32_t as_int<float>(float v) {
  return __float2int_rn(v);
}

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

struct EpiDev {
  int mode;
  const float* bias_f;
  int act;
  float clip_lo, clip_hi;
  const float* slope;  // act 4 (PRelu): one slope per output channel
  int round_tf32;
  const float* residual;
  const int32_t* bias_i;
  int x_zp;
  const float* x_zp_dev;
  const int32_t* x_zp_rows;
  const int32_t* w_zp;
  int n_w_zp;
  const float* combined;
  int y_zp, lo, hi;
  DT out_dt;
  const float* dq_w_scale;
  const float* dq_x_scale;
  const float* dq_bias;
  int dq_act;
};

__device__ __forceinline__ void store_int(void* out, DT dt, int64_t idx, int32_t q) {
  switch (dt) {
    case DT::U8: ((uint8_t*)out)[idx] = (uint8_t)q; break;
    case DT::I8: ((int8_t*)out)[idx] = (int8_t)q; break;
    case DT::I16: ((int16_t*)out)[idx] = (int16_t)q; break;
    case DT::I32: ((int32_t*)out)[idx] = q; break;
    default: ((float*)out)[idx] = (float)q; break;
  }
}

__device__ __forceinline__ float erf_poly(float x) {  // nn_ops/activations.rs:578, same operation order
  const float sign = x >= 0.0f ? 1.0f : -1.0f;
  x = fabsf(x);
  const float t = __fdiv_rn(1.0f, __fadd_rn(1.0f, __fmul_rn(0.3275911f, x)));
  float p = __fadd_rn(-1.4531521f, __fmul_rn(t, 1.0614054f));
  p = __fadd_rn(1.4214138f, __fmul_rn(t, p));
  p = __fadd_rn(-0.28449672f, __fmul_rn(t, p));
  p = __fadd_rn(0.2548296f, __fmul_rn(t, p));
  return __fmul_rn(sign, __fsub_rn(1.0f, __fmul_rn(__fmul_rn(t, p), expf(__fmul_rn(-x, x)))));
}

__device__ __forceinline__ void finish_int(const EpiDev& e, void* out, int64_t idx, int oc, long long acc) {
  if (e.mode == EPI_DEQUANT) {
    const long long c = acc < -2147483648LL ? -2147483648LL : (acc > 2147483647LL ? 2147483647LL : acc);
    float y = __fadd_rn(__fmul_rn(__int2float_rn((int)c), __fmul_rn(*e.dq_x_scale, e.dq_w_scale[oc])), e.dq_bias[oc]);
    if (e.dq_act == 1) y = __fmul_rn(__fmul_rn(y, 0.5f), __fadd_rn(1.0f, erf_poly(__fmul_rn(y, 0.70710678118654752440f))));
    if (e.dq_act == 2) {
      const float inner = __fmul_rn(0.7978846f, __fadd_rn(y, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, y), y), y)));
      y = __fmul_rn(__fmul_rn(0.5f, y), __fadd_rn(1.0f, tanhf(inner)));
    }
    if (e.round_tf32) y = round_tf32(y);
    ((float*)out)[idx] = y;
    return;
  }
  if (e.mode == EPI_INT32) {
    long long c = acc < -2147483648LL ? -2147483648LL : (acc > 2147483647LL ? 2147483647LL : acc);
    store_int(out, e.out_dt, idx, (int32_t)c);
    return;
  }
  // f64 product and f64 add, each rounded once; then round-to-nearest-even and saturate
  // (SatRange::requantize, quant_ops/mod.rs:229-233).
  double scaled = __dadd_rn(__dmul_rn((double)acc, (double)e.combined[oc]), (double)e.y_zp);
  double r = rint(scaled);
  r = fmin(fmax(r, (double)e.lo), (double)e.hi);
  store_int(out, e.out_dt, idx, (int32_t)r);
}

template <typename TX, typename TW, bool IS_INT>
__global__ void conv_direct_kernel(const TX* __restrict__ x, const TW* __restrict__ w, void* __restrict__ out, ConvShape cs, EpiDev e,
                                   int x_plain_nchw, int64_t total) {
  const int cg = cs.C / cs.group, ocg = cs.OC / cs.group;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    int oc = (int)(idx % cs.OC);
    int64_t m = idx / cs.OC;
    int q = (int)(m % cs.Q);
    int64_t t = m / cs.Q;
    int p = (int)(t % cs.P);
    int64_t n = t / cs.P;
    int g = oc / ocg;
    if (IS_INT) {
      long long acc = e.bias_i ? (long long)e.bias_i[oc] : 0;
      int xz = e.x_zp_dev ? __float2int_rn(*e.x_zp_dev) : e.x_zp;
      if (e.x_zp_rows) xz = e.x_zp_rows[m];
      int wz = e.n_w_zp > 1 ? e.w_zp[oc] : (e.n_w_zp == 1 ? e.w_zp[0] : 0);
      for (int r = 0; r < cs.R; ++r) {
        int ih = p * cs.sh + r * cs.dh - cs.pt;
        if (ih < 0 || ih >= cs.H) continue;
        for (int s = 0; s < cs.S; ++s) {
          int iw = q * cs.sw + s * cs.dw - cs.pl;
          if (iw < 0 || iw >= cs.W) continue;
          const TW* wp = w + ((int64_t)(r * cs.S + s) * cg) * cs.OC + oc;
          if (x_plain_nchw) {
            const TX* xp = x + ((n * cs.C + (int64_t)g * cg) * cs.H + ih) * cs.W + iw;
            for (int ic = 0; ic < cg; ++ic)
              acc += (long long)(as_int(xp[(int64_t)ic * cs.H * cs.W]) - xz) * (long long)(as_int(wp[(int64_t)ic * cs.OC]) - wz);
          } else {
            const TX* xp = x + ((n * cs.H + ih) * cs.W + iw) * cs.C + (int64_t)g * cg;
            for (int ic = 0; ic < cg; ++ic) acc += (long long)(as_int(xp[ic]) - xz) * (long long)(as_int(wp[(int64_t)ic * cs.OC]) - wz);
          }
        }
      }
      finish_int(e, out, idx, oc, acc);
    } else {
      float acc = 0.f;
      for (int r = 0; r < cs.R; ++r) {
        int ih = p * cs.sh + r * cs.dh - cs.pt;
        if (ih < 0 || ih >= cs.H) continue;
        for (int s = 0; s < cs.S; ++s) {
          int iw = q * cs.sw + s * cs.dw - cs.pl;
          if (iw < 0 || iw >= cs.W) continue;
          const TW* wp = w + ((int64_t)(r * cs.S + s) * cg) * cs.OC + oc;
          if (x_plain_nchw) {
            const TX* xp = x + ((n * cs.C + (int64_t)g * cg) * cs.H + ih) * cs.W + iw;
            for (int ic = 0; ic < cg; ++ic) acc = fmaf((float)xp[(int64_t)ic * cs.H * cs.W], (float)wp[(int64_t)ic * cs.OC], acc);
          } else {
            const TX* xp = x + ((n * cs.H + ih) * cs.W + iw) * cs.C + (int64_t)g * cg;
            for (int ic = 0; ic < cg; ++ic) acc = fmaf((float)xp[ic], (float)wp[(int64_t)ic * cs.OC], acc);
          }
        }
      }
      float v = e.bias_f ? acc + e.bias_f[oc] : acc;
      if (e.residual) v = __fadd_rn(v, e.residual[idx]);
      if (e.act == 1) v = fmaxf(v, 0.f);
      else if (e.act == 2) v = fminf(fmaxf(v, e.clip_lo), e.clip_hi);
      else if (e.act == 3) v = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));  // silu
      else if (e.act == 4) v = v >= 0.f ? v : __fmul_rn(v, e.slope[oc]);  // prelu
      if (e.round_tf32) v = round_tf32(v);
      ((float*)out)[idx] = v;
    }
  }
}

__global__ void matmul_f32_direct_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, int64_t M, int64_t K,
                                         int64_t N, int64_t a_bs, int64_t b_bs) {
  // 32x32 output tile per block, K stepped through shared memory in slabs of 32.
  __shared__ float As[32][33], Bs[32][33];
  int64_t batch = blockIdx.z;
  const float* A = a + batch * a_bs;
  const float* B = b + batch * b_bs;
  float* C = c + batch * M * N;
  int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  int64_t row0 = (int64_t)blockIdx.y * 32, col0 = (int64_t)blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t k0 = 0; k0 < K; k0 += 32) {
    for (int i = ty; i < 32; i += 8) {
      int64_t r = row0 + i, kk = k0 + tx;
      As[i][tx] = (r < M && kk < K) ? A[r * K + kk] : 0.f;
      int64_t kr = k0 + i, cc = col0 + tx;
      Bs[i][tx] = (kr < K && cc < N) ? B[kr * N + cc] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int i = ty + j * 8;
      float s = acc[j];
      for (int kk = 0; kk < 32; ++kk) s = fmaf(As[i][kk], Bs[kk][tx], s);
      acc[j] = s;
    }
    __syncthreads();
  }
  for (int j = 0; j < 4; ++j) {
    int64_t r = row0 + ty + j * 8, cc = col0 + tx;
    if (r < M && cc < N) C[r * N + cc] = acc[j];
  }
}

template <typename TX, typename TW, bool IS_INT>
void launch_conv(const void* x, const void* w, void* out, const ConvShape& cs, const EpiDev& e, int x_plain_nchw, cudaStream_t s) {
  int64_t total = cs.M() * cs.OC;
  if (total == 0) return;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 256) blocks = 148 * 256;
  conv_direct_kernel<TX, TW, IS_INT><<<(unsigned)blocks, 256, 0, s>>>((const TX*)x, (const TW*)w, out, cs, e, x_plain_nchw, total);
}

}  // namespace

void conv_direct(const void* x, DT x_dt, int x_plain_nchw, const void* w, DT w_dt, void* out, const ConvShape& cs, const Epilogue& ep,
                 cudaStream_t s) {
  EpiDev e{ep.mode,     ep.bias_f,    ep.act,  ep.clip_lo, ep.clip_hi,  ep.slope, ep.round_tf32, ep.residual, ep.bias_i, ep.x_zp, ep.x_zp_dev,
           ep.x_zp_rows, ep.w_zp,     ep.n_w_zp, ep.combined, ep.y_zp,  ep.relu_fused && ep.lo < 0 ? 0 : ep.lo, ep.hi, ep.out_dt, ep.dq_w_scale, ep.dq_x_scale_dev, ep.dq_bias, ep.dq_act};
  if (ep.mode == EPI_F32) {
    if (x_dt != DT::F32 || w_dt != DT::F32) OXB_FAIL("conv_direct: float epilogue needs f32 operands");
    launch_conv<float, float, false>(x, w, out, cs, e, x_plain_nchw, s);
    return;
  }
#define OXB_DISPATCH_W(TX)                                                                    \
  switch (w_dt) {                                                                             \
    case DT::I8: launch_conv<TX, int8_t, true>(x, w, out, cs, e, x_plain_nchw, s); return;    \
    case DT::U8: launch_conv<TX, uint8_t, true>(x, w, out, cs, e, x_plain_nchw, s); return;   \
    case DT::I16: launch_conv<TX, int16_t, true>(x, w, out, cs, e, x_plain_nchw, s); return;  \
    case DT::I32: launch_conv<TX, int32_t, true>(x, w, out, cs, e, x_plain_nchw, s); return;  \
    default: break;                                                                           \
  }
  switch (x_dt) {
    case DT::U8: OXB_DISPATCH_W(uint8_t) break;
    case DT::I8: OXB_DISPATCH_W(int8_t) break;
    case DT::I16: OXB_DISPATCH_W(int16_t) break;
    case DT::I32: OXB_DISPATCH_W(int32_t) break;
    default: break;
  }
#undef OXB_DISPATCH_W
  OXB_FAIL("conv_direct: unsupported operand storage types (%s x %s)", dt_name(x_dt), dt_name(w_dt));
}

void matmul_f32_direct(const float* a, const float* b, float* c, int64_t batch, int64_t M, int64_t K, int64_t N, int64_t a_bstride,
                       int64_t b_bstride, cudaStream_t s) {
  if (batch * M * N == 0) return;
  dim3 block(32, 8), grid((unsigned)ceil_div(N, 32), (unsigned)ceil_div(M, 32), (unsigned)batch);
  matmul_f32_direct_kernel<<<grid, block, 0, s>>>(a, b, c, M, K, N, a_bstride, b_bstride);
}

}  // namespace k
}  // namespace oxb
