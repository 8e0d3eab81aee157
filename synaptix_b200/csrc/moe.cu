// A mixture of gated feed-forward experts (sm_100a), float32 and bfloat16; router, softmax and weights are 32-bit.
//
//   moe_route_kernel   one block a token: logits z_e = Wr[e] . x in 32-bit (Wr float32, x widened), softmax over ALL
//                      experts, the `top` largest scores (ties: the lower index), weights = score / (sum of the chosen
//                      + sum_eps) * scale  -> ids [T, top], weights [T, top]
//   moe_sort_kernel    one block: the T * top (token, choice) pairs sorted by expert: offsets [E + 1], order [T * top]
//                      (sorted place -> pair), place [T * top] (pair -> sorted place).  The order inside an expert's
//                      group is whatever the atomics give; no result depends on it (each row is computed alone).
//   moe_gemm_kernel    grouped product: tile i of the grid's y axis belongs to the expert whose rows hold it (a block
//                      finds it from `offsets`; tiles beyond the last return).  GATE_UP: rows are gathered from x by
//                      pair / top, the expert's [gate; up] matrix gives two accumulators and the result is
//                      silu(gate) * up  [T * top, ff] in sorted order; else rows are read in sorted order and the
//                      result is the plain product [T * top, N].  64x64x16 tiles, 4x4 results a thread, 32-bit FFMA.
//   moe_combine_kernel out[t] = sum_j weights[t, j] * y[place[t * top + j]], the choices in their order.
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024

template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ wr, int W, int E,
                                                        int top, float scale, float sum_eps, int* __restrict__ ids,
                                                        float* __restrict__ weights) {
  extern __shared__ float sm[];
  float* xs = sm;            // W
  float* z = sm + W;         // E
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < W; i += 128) xs[i] = to_f32(x[(size_t)t * W + i]);
  __syncthreads();
  for (int e = warp; e < E; e += 4) {
    const float* w = wr + (size_t)e * W;
    float d = 0.f;
    for (int i = lane; i < W; i += 32) d = fmaf(xs[i], w[i], d);
    d = warp_sum(d);
    if (lane == 0) z[e] = d;
  }
  __syncthreads();
  if (warp != 0) return;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - mx); z[e] = p; sum += p; }
  sum = warp_sum(sum);
  __syncwarp();
  float chosen_sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float p = z[e];
      if (p > best) { best = p; bi = e; }       // a lane walks upwards: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    const float s = best / sum;
    chosen_sum += s;
    if (lane == 0) {
      ids[(size_t)t * top + j] = bi;
      weights[(size_t)t * top + j] = s;
      z[bi] = -2.f;                             // taken
    }
    __syncwarp();
  }
  const float f = scale / (chosen_sum + sum_eps);
  for (int j = lane; j < top; j += 32) weights[(size_t)t * top + j] *= f;
}

extern "C" int sx_moe_route(const void* x, const float* wr, int T, int W, int E, int top, float scale, float sum_eps,
                            int* ids, float* weights, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || W <= 0) return SX_ERR_SIZE;
  const size_t smem = (size_t)(W + E) * sizeof(float);
  if (smem > 96 * 1024) return SX_ERR_SIZE;
  if (dt == SX_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(moe_route_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)x, wr, W, E, top, scale, sum_eps, ids, weights);
  }
  if (dt == SX_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(moe_route_kernel<bf16>, dim3(T), dim3(128), smem, stream, (const bf16*)x, wr, W, E, top, scale, sum_eps, ids, weights);
  }
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ offsets,
                                                        int* __restrict__ order, int* __restrict__ place) {
  __shared__ int count[MOE_MAX_EXPERTS];
  __shared__ int start[MOE_MAX_EXPERTS + 1];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) count[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (tid == 0) {
    int s = 0;
    for (int e = 0; e < E; ++e) { start[e] = s; s += count[e]; }
    start[E] = s;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += 1024) offsets[e] = start[e];
  for (int e = tid; e < E; e += 1024) count[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    const int p = start[e] + atomicAdd(&count[e], 1);
    order[p] = i;
    place[i] = p;
  }
}

extern "C" int sx_moe_sort(const int* ids, int n, int E, int* offsets, int* order, int* place, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS) return SX_ERR_SIZE;
  return sx_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, ids, n, E, offsets, order, place);
}

// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float moe_silu(float g) { return g / (1.f + expf(-g)); }

template <typename TA, typename TW, typename TC, bool GATE_UP>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ Wt, TC* __restrict__ C,
                                                       const int* __restrict__ offsets, const int* __restrict__ order,
                                                       int E, int N, int K, int top) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[GATE_UP ? BK : 1][BN + 4];
  __shared__ int src[BM];
  __shared__ int which[3];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  if (tid == 0) {
    // the tile's expert and first row: tiles are counted expert by expert
    int tile = blockIdx.y, e = 0, r0 = -1;
    for (; e < E; ++e) {
      const int n_e = offsets[e + 1] - offsets[e];
      const int tiles = (n_e + BM - 1) / BM;
      if (tile < tiles) { r0 = offsets[e] + tile * BM; break; }
      tile -= tiles;
    }
    which[0] = e; which[1] = r0; which[2] = r0 >= 0 ? min(BM, offsets[e + 1] - r0) : 0;
  }
  __syncthreads();
  const int e = which[0], r0 = which[1], nr = which[2];
  if (r0 < 0) return;
  if (tid < BM) src[tid] = tid < nr ? (GATE_UP ? order[r0 + tid] / top : r0 + tid) : -1;
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * BN;
  const int NW = GATE_UP ? 2 * N : N;         // rows of an expert's matrix
  const TW* We = Wt + (size_t)e * NW * K;
  float acc[4][4], acu[GATE_UP ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GATE_UP) acu[i][j] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = idx & 15;
      const int k = k0 + c;
      const int m = src[r], n = n0 + r;
      As[c][r] = (m >= 0 && k < K) ? to_f32(A[(size_t)m * K + k]) : 0.f;
      Ws[c][r] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
      if (GATE_UP) Us[c][r] = (n < N && k < K) ? to_f32(We[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = Ws[kk][tx * 4 + j]; if (GATE_UP) u[j] = Us[kk][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATE_UP) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= nr) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)(r0 + r) * N + n] = from_f32<TC>(GATE_UP ? moe_silu(acc[i][j]) * acu[i][j] : acc[i][j]);
    }
  }
}

// rows: T * top; the grid's y axis has room for every expert's last, partly filled tile
extern "C" int sx_moe_gemm(const void* A, const void* Wt, void* C, const int* offsets, const int* order, int rows, int E, int N,
                           int K, int top, int gate_up, int a_dt, int c_dt, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || N <= 0 || K <= 0) return SX_ERR_SIZE;
  const int tiles = (rows + 63) / 64 + (E < rows ? E : rows);
  if (tiles > 65535) return SX_ERR_SIZE;
  dim3 grid((N + 63) / 64, tiles);
#define MOE_GO(TA, TC, GU) return sx_launch(moe_gemm_kernel<TA, TA, TC, GU>, grid, dim3(256), 0, stream, (const TA*)A, (const TA*)Wt, (TC*)C, offsets, order, E, N, K, top)
  if (gate_up) {
    if (a_dt == SX_F32 && c_dt == SX_F32) MOE_GO(float, float, true);
    if (a_dt == SX_BF16 && c_dt == SX_BF16) MOE_GO(bf16, bf16, true);
  } else {
    if (a_dt == SX_F32 && c_dt == SX_F32) MOE_GO(float, float, false);
    if (a_dt == SX_BF16 && c_dt == SX_F32) MOE_GO(bf16, float, false);
    if (a_dt == SX_BF16 && c_dt == SX_BF16) MOE_GO(bf16, bf16, false);
  }
#undef MOE_GO
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
template <typename TY, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   TO* __restrict__ out, int W, int top) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < top; ++j)
      s = fmaf(weights[(size_t)t * top + j], to_f32(y[(size_t)place[(size_t)t * top + j] * W + c]), s);
    out[(size_t)t * W + c] = from_f32<TO>(s);
  }
}

extern "C" int sx_moe_combine(const void* y, int y_dt, const int* place, const float* weights, void* out, int out_dt, int T,
                              int W, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (y_dt == SX_F32 && out_dt == SX_F32)
    return sx_launch(moe_combine_kernel<float, float>, dim3(T), dim3(256), 0, stream, (const float*)y, place, weights, (float*)out, W, top);
  if (y_dt == SX_F32 && out_dt == SX_BF16)
    return sx_launch(moe_combine_kernel<float, bf16>, dim3(T), dim3(256), 0, stream, (const float*)y, place, weights, (bf16*)out, W, top);
  if (y_dt == SX_BF16 && out_dt == SX_BF16)
    return sx_launch(moe_combine_kernel<bf16, bf16>, dim3(T), dim3(256), 0, stream, (const bf16*)y, place, weights, (bf16*)out, W, top);
  return SX_ERR_DTYPE;
}
