// Kernels of a block whose branches read the same residual stream (sm_100a), float32 and bfloat16.
//
//   add_scaled_rmsnorm: v = h[t] + sa * a[t] + sb * b[t] (sa, sb vectors over the width, each term optional);
//                       if write_h: h[t] = v;  y1[r] = v * rsqrt(mean(v^2) + eps) * g1;  y2[r] = ... * g2 (optional).
//                       Rows: r = 0..R-1, t = rows ? rows[r] : r.  One block a row; the row stays in shared memory
//                       between the sum of squares and the outputs, so memory is passed over once.
//   add_scaled:         h[t] += sa * a[t] + sb * b[t]        (no norm behind it)
//   scale_rows:         x *= s                               (float32, in place: logits)
// The stream, the factors, the gains and all sums are 32-bit; a and b may each be float32 or bfloat16.
#include "common.cuh"

__device__ __forceinline__ float ld_any(const void* p, int dt, size_t i) {
  return dt == SX_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

__device__ __forceinline__ float4 ld_any4(const void* p, int dt, size_t i) {      // four elements from a 4-aligned place
  if (dt == SX_F32) return *reinterpret_cast<const float4*>((const float*)p + i);
  const uint2 v = *reinterpret_cast<const uint2*>((const bf16*)p + i);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename TO> __device__ __forceinline__ void st4(TO* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

// VEC4: the width is a multiple of 4 and every array 16-byte aligned: four elements a load
template <typename TO, bool VEC4>
__global__ void __launch_bounds__(256) add_scaled_rmsnorm_kernel(
    float* __restrict__ h, const void* __restrict__ a, int a_dt, const float* __restrict__ sa,
    const void* __restrict__ b, int b_dt, const float* __restrict__ sb, const float* __restrict__ g1,
    const float* __restrict__ g2, float eps, TO* __restrict__ y1, TO* __restrict__ y2, const int* __restrict__ rows,
    int H, int write_h) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* hr = h + (size_t)t * H;
  float ss = 0.f;
  if (VEC4) {
#pragma unroll 2
    for (int i = threadIdx.x * 4; i < H; i += 1024) {
      float4 v = *reinterpret_cast<const float4*>(hr + i);
      if (a || b) {
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a) {
          d = ld_any4(a, a_dt, (size_t)t * H + i);
          if (sa) { const float4 f = *reinterpret_cast<const float4*>(sa + i); d.x *= f.x; d.y *= f.y; d.z *= f.z; d.w *= f.w; }
        }
        if (b) {
          float4 e = ld_any4(b, b_dt, (size_t)t * H + i);
          if (sb) { const float4 f = *reinterpret_cast<const float4*>(sb + i); e.x *= f.x; e.y *= f.y; e.z *= f.z; e.w *= f.w; }
          d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
        }
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (write_h) *reinterpret_cast<float4*>(hr + i) = v;
      }
      *reinterpret_cast<float4*>(row + i) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i];
      if (a || b) {
        float d = 0.f;
        if (a) d = ld_any(a, a_dt, (size_t)t * H + i) * (sa ? sa[i] : 1.f);
        if (b) d += ld_any(b, b_dt, (size_t)t * H + i) * (sb ? sb[i] : 1.f);
        v += d;
        if (write_h) hr[i] = v;
      }
      row[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (VEC4) {
#pragma unroll 2
    for (int i = threadIdx.x * 4; i < H; i += 1024) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      const float4 f = *reinterpret_cast<const float4*>(g1 + i);
      st4<TO>(y1 + (size_t)r * H + i, make_float4(v.x * inv * f.x, v.y * inv * f.y, v.z * inv * f.z, v.w * inv * f.w));
      if (y2) {
        const float4 k = *reinterpret_cast<const float4*>(g2 + i);
        st4<TO>(y2 + (size_t)r * H + i, make_float4(v.x * inv * k.x, v.y * inv * k.y, v.z * inv * k.z, v.w * inv * k.w));
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = row[i] * inv;
      y1[(size_t)r * H + i] = from_f32<TO>(v * g1[i]);
      if (y2) y2[(size_t)r * H + i] = from_f32<TO>(v * g2[i]);
    }
  }
}

template <typename TO, bool VEC4>
static int add_scaled_rmsnorm_go(float* h, const void* a, int a_dt, const float* sa, const void* b, int b_dt, const float* sb,
                                 const float* g1, const float* g2, float eps, void* y1, void* y2, const int* rows, int R, int H,
                                 int write_h, cudaStream_t stream) {
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(add_scaled_rmsnorm_kernel<TO, VEC4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return sx_launch(add_scaled_rmsnorm_kernel<TO, VEC4>, dim3(R), dim3(256), smem, stream, h, a, a_dt, sa, b, b_dt, sb, g1, g2, eps,
                   (TO*)y1, (TO*)y2, rows, H, write_h);
}

extern "C" int sx_add_scaled_rmsnorm(float* h, const void* a, int a_dt, const float* sa, const void* b, int b_dt,
                                     const float* sb, const float* g1, const float* g2, float eps, void* y1, void* y2,
                                     const int* rows, int R, int H, int out_dt, int write_h, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || H > 24576) return SX_ERR_SIZE;
  const uintptr_t all = (uintptr_t)h | (uintptr_t)a | (uintptr_t)sa | (uintptr_t)b | (uintptr_t)sb | (uintptr_t)g1 | (uintptr_t)g2 |
                        (uintptr_t)y1 | (uintptr_t)y2;
  const bool vec = (H % 4 == 0) && (all % 16 == 0);
#define AS_GO(TO, V) return add_scaled_rmsnorm_go<TO, V>(h, a, a_dt, sa, b, b_dt, sb, g1, g2, eps, y1, y2, rows, R, H, write_h, stream)
  if (out_dt == SX_F32) { if (vec) AS_GO(float, true); AS_GO(float, false); }
  if (out_dt == SX_BF16) { if (vec) AS_GO(bf16, true); AS_GO(bf16, false); }
#undef AS_GO
  return SX_ERR_DTYPE;
}

__global__ void add_scaled_kernel(float* __restrict__ h, const void* __restrict__ a, int a_dt, const float* __restrict__ sa,
                                  const void* __restrict__ b, int b_dt, const float* __restrict__ sb, int H, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % H);
  float d = 0.f;
  if (a) d = ld_any(a, a_dt, i) * (sa ? sa[c] : 1.f);
  if (b) d += ld_any(b, b_dt, i) * (sb ? sb[c] : 1.f);
  h[i] += d;
}

extern "C" int sx_add_scaled(float* h, const void* a, int a_dt, const float* sa, const void* b, int b_dt, const float* sb,
                             int T, int H, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  const size_t n = (size_t)T * H;
  return sx_launch(add_scaled_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, h, a, a_dt, sa, b, b_dt, sb, H, n);
}

__global__ void scale_rows_kernel(float* __restrict__ x, float s, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

extern "C" int sx_scale_rows(float* x, long long n, float s, cudaStream_t stream) {
  if (n <= 0) return 0;
  return sx_launch(scale_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, s, (size_t)n);
}
