// RMSNorm forward and backward over rows of 16-bit elements.
//
// Forward replaces rmsnorm_twoPassAlgo_e8 (kernel_src/csrc/rms_norm/rms_norm_cutlass.cu:80-156):
//   s_row = rsqrt(mean(x^2) + eps) in fp32, written to rms_out;  out = T(float(x) * s_row * float(w)).
// The reference reads every row twice (once for the sum, once for the output); here a row is read
// once into registers (up to 16384 columns; wider rows take the two-pass route), so the launch
// moves the compulsory bytes only: one read and one write of [rows, cols].
//
// Backward replaces the torch expressions of src/loquetier_src/kernel_utils.py:166-176:
//   dW = sum_rows(x * s * gO)          dX = (gO * w - x * dot * s^2 / cols) * s,  dot = sum_cols(gO * w * x)
// in one pass over x and gO (the reference makes about ten elementwise passes): persistent CTAs walk
// rows with a fixed stride, keep their share of dW in fp32 registers and park it in the caller's
// workspace; a second small kernel adds the parked partials in a fixed order (deterministic).
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kRmsThreads = 256;  // threads of the dW kernel and the narrowest row kernels

// Sum over the CTA (NT threads), the same value in every thread.
template <int NT>
__device__ __forceinline__ float rms_block_sum(float v, float* red) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < NT / 32 ? red[lane] : 0.f;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
  return t;
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack2<T>(u.x), b = unpack2<T>(u.y), c = unpack2<T>(u.z), d = unpack2<T>(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
}

// VPT: 16-byte chunks per thread held in registers (rows of up to 8 * VPT * NT columns); 0 = wider rows,
// read twice instead.  Wide rows get more threads rather than more registers per thread, so that several
// CTAs stay resident and hide each other's latency.
template <typename T, int VPT, int NT>
__global__ void __launch_bounds__(NT) rms_norm_fwd_kernel(uint4* __restrict__ out, float* __restrict__ rms_out,
                                                                   const uint4* __restrict__ x,
                                                                   const uint4* __restrict__ w, int rows, int n8,
                                                                   float inv_n, float eps) {
  __shared__ float red[32];
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  constexpr int V = VPT > 0 ? VPT : 1;
  uint4 wv[V];
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = tid + i * NT;
      wv[i] = c < n8 ? __ldg(w + c) : make_uint4(0, 0, 0, 0);
    }
  }
  if (VPT > 0) {
    // the next row is requested before the current one is reduced, so that a CTA always has a row in flight
    uint4 xv[V], xn[V];
    auto load_row = [&](int row, uint4 (&dst)[V]) {
      const uint4* xr = x + static_cast<size_t>(row) * n8;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int c = tid + i * NT;
        dst[i] = (row < rows && c < n8) ? __ldcs(xr + c) : make_uint4(0, 0, 0, 0);
      }
    };
    load_row(blockIdx.x, xv);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      load_row(row + gridDim.x, xn);
      uint4* orow = out + static_cast<size_t>(row) * n8;
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float f[8];
        unpack8<T>(xv[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
      }
      const float s = rsqrtf(rms_block_sum<NT>(ss, red) * inv_n + eps);
      if (tid == 0) rms_out[row] = s;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int c = tid + i * NT;
        if (c < n8) {
          float f[8], g[8];
          unpack8<T>(xv[i], f);
          unpack8<T>(wv[i], g);
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = f[k] * s * g[k];
          __stcs(orow + c, pack8<T>(f));
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) xv[i] = xn[i];
    }
  } else {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const uint4* xr = x + static_cast<size_t>(row) * n8;
      uint4* orow = out + static_cast<size_t>(row) * n8;
      float ss = 0.f;
      for (int c = tid; c < n8; c += NT) {
        float f[8];
        unpack8<T>(__ldg(xr + c), f);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
      }
      const float s = rsqrtf(rms_block_sum<NT>(ss, red) * inv_n + eps);
      if (tid == 0) rms_out[row] = s;
      for (int c = tid; c < n8; c += NT) {
        float f[8], g[8];
        unpack8<T>(__ldg(xr + c), f);
        unpack8<T>(__ldg(w + c), g);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = f[k] * s * g[k];
        __stcs(orow + c, pack8<T>(f));
      }
    }
  }
}

// dX per row and this CTA's share of dW (fp32, parked at partial[blockIdx.x][cols]).
template <typename T, int VPT, int NT>
__global__ void __launch_bounds__(NT) rms_norm_bwd_kernel(uint4* __restrict__ dx, float* __restrict__ partial,
                                                                   const uint4* __restrict__ go,
                                                                   const uint4* __restrict__ x,
                                                                   const uint4* __restrict__ w,
                                                                   const float* __restrict__ rms, int rows, int n8,
                                                                   float inv_n) {
  __shared__ float red[32];
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  constexpr int V = VPT > 0 ? VPT : 1;
  float* prow = partial + static_cast<size_t>(blockIdx.x) * n8 * 8;
  if (VPT > 0) {
    uint4 wv[V];
    float acc[V][8];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = tid + i * NT;
      wv[i] = c < n8 ? __ldg(w + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
    }
    // the next row is requested before the current one is reduced, so that a CTA always has a row in flight
    uint4 xv[V], gv[V], xn[V], gn[V];
    auto load_row = [&](int row, uint4 (&dx_)[V], uint4 (&dg_)[V]) {
      const uint4* xr = x + static_cast<size_t>(row) * n8;
      const uint4* gr = go + static_cast<size_t>(row) * n8;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int c = tid + i * NT;
        const bool ok = row < rows && c < n8;
        dx_[i] = ok ? __ldcs(xr + c) : make_uint4(0, 0, 0, 0);
        dg_[i] = ok ? __ldcs(gr + c) : make_uint4(0, 0, 0, 0);
      }
    };
    load_row(blockIdx.x, xv, gv);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      load_row(row + gridDim.x, xn, gn);
      const float s = rms[row];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float xf[8], gf[8], wf[8];
        unpack8<T>(xv[i], xf);
        unpack8<T>(gv[i], gf);
        unpack8<T>(wv[i], wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot += gf[k] * wf[k] * xf[k];
          acc[i][k] += xf[k] * s * gf[k];
        }
      }
      dot = rms_block_sum<NT>(dot, red);
      const float coef = dot * s * s * inv_n;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int c = tid + i * NT;
        if (c < n8) {
          float xf[8], gf[8], wf[8];
          unpack8<T>(xv[i], xf);
          unpack8<T>(gv[i], gf);
          unpack8<T>(wv[i], wf);
#pragma unroll
          for (int k = 0; k < 8; ++k) xf[k] = (gf[k] * wf[k] - xf[k] * coef) * s;
          __stcs(dx + static_cast<size_t>(row) * n8 + c, pack8<T>(xf));
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        xv[i] = xn[i];
        gv[i] = gn[i];
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = tid + i * NT;
      if (c < n8) {
        *reinterpret_cast<float4*>(prow + c * 8) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(prow + c * 8 + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
  } else {
    // wide rows: dW shares live in the workspace itself (this CTA's own row of it)
    for (int c = tid; c < n8 * 8; c += NT) prow[c] = 0.f;
    __syncthreads();
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const uint4* xr = x + static_cast<size_t>(row) * n8;
      const uint4* gr = go + static_cast<size_t>(row) * n8;
      const float s = rms[row];
      float dot = 0.f;
      for (int c = tid; c < n8; c += NT) {
        float xf[8], gf[8], wf[8];
        unpack8<T>(__ldg(xr + c), xf);
        unpack8<T>(__ldg(gr + c), gf);
        unpack8<T>(__ldg(w + c), wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot += gf[k] * wf[k] * xf[k];
          prow[c * 8 + k] += xf[k] * s * gf[k];
        }
      }
      dot = rms_block_sum<NT>(dot, red);
      const float coef = dot * s * s * inv_n;
      for (int c = tid; c < n8; c += NT) {
        float xf[8], gf[8], wf[8];
        unpack8<T>(__ldg(xr + c), xf);
        unpack8<T>(__ldg(gr + c), gf);
        unpack8<T>(__ldg(w + c), wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) xf[k] = (gf[k] * wf[k] - xf[k] * coef) * s;
        __stcs(dx + static_cast<size_t>(row) * n8 + c, pack8<T>(xf));
      }
    }
  }
}

// dW[col] = sum over the parked partials in index order.  A CTA owns 32 columns: warp w adds the
// partials w, w + 8, ... and the eight warp sums are added in warp order.
template <typename T>
__global__ void __launch_bounds__(kRmsThreads) rms_norm_dw_kernel(void* __restrict__ dw,
                                                                  const float* __restrict__ partial, int nparts,
                                                                  int cols, int dw_fp32) {
  __shared__ float red[kRmsThreads / 32][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  pdl_wait();
  pdl_trigger();
  float s = 0.f;
  if (col < cols)
    for (int p = warp; p < nparts; p += kRmsThreads / 32) s += __ldcg(partial + static_cast<size_t>(p) * cols + col);
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && col < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kRmsThreads / 32; ++i) t += red[i][lane];
    if (dw_fp32) static_cast<float*>(dw)[col] = t;
    else static_cast<T*>(dw)[col] = static_cast<T>(t);
  }
}

}  // namespace smlm
