// The matrix memory with exponential gates (mLSTM) for sm_100a, float32 and bfloat16 inputs; gates, states, decays,
// exponentials, norms and all sums are 32-bit in both.
//
// Per head, with q (times q_scale), k of D and v of Dv elements and the gates' pre-activations zi, zf (32-bit, biases
// added here):
//   i = cap tanh(zi / cap),  f = logsigmoid(cap tanh(zf / cap)),
//   m_t = max(f + m_(t-1), i),  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,  n_t likewise with k alone,
//   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps),
//   out = o_t / sqrt(mean(o_t^2) + eps) * gain * sigmoid(g)      (mean over the head's Dv elements)
// S [slots, H, D, Dv], n [slots, H, D] and m [slots, H] are each sequence's state, moved on.
//
//   mlstm_walk_kernel   one block a (head, sequence) walks the tokens one after the other with S in shared memory
//                       (single-token steps, short portions, and sizes the pieces do not take).
//   pieces of 64 tokens (long portions):
//   mlstm_gates_kernel  a block a (head, sequence): the gates of all tokens, the running sums b of f inside each piece,
//                       each piece's own maximum m_loc = max_j (b_end - b_j + i_j), and then, one after the other
//                       over the pieces, the maximum m at every piece's begin (m_end = max(b_end + m_begin, m_loc)).
//   mlstm_piece_kernel  a block a (piece, head, sequence): U = sum_j exp(b_end - b_j + i_j - m_loc) k_j v_j^T and the
//                       same sum of k_j alone.
//   mlstm_carry_kernel  a block a (head, sequence) and slice of the state: the state at every piece's begin,
//                       S_end = exp(b_end + m_begin - m_end) S_begin + exp(m_loc - m_end) U, one piece after the other;
//                       the last one is the sequence's new state.
//   mlstm_apply_kernel  a block a (piece, head, sequence): with m_i = max(b_i + m_begin, max_{j<=i} (b_i - b_j + i_j)),
//                       num_i = exp(b_i + m_begin - m_i) S_begin^T q_i + sum_{j<=i} exp(b_i - b_j + i_j - m_i) (q_i . k_j) v_j,
//                       the denominator's dot product likewise with n_begin and without v; unit norm, gain, gate.
#include "common.cuh"

#define ML_THREADS 256
#define ML_PIECE 64

__device__ __forceinline__ float ml_cap(float z, float cap) { return cap * tanhf(z / cap); }
__device__ __forceinline__ float ml_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float ml_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }

struct MlArgs {
  const void* proj;            // [T, row]
  int row, q_off, k_off, v_off, g_off;
  const float* gates;          // [T, 2H]: zi of every head, then zf
  const float* bias;           // [2H]
  float cap, q_scale, eps, den_eps;
  const float* gain;           // [H * Dv]
  float* S;                    // [slots, H, D, Dv]
  float* n;                    // [slots, H, D]
  float* m;                    // [slots, H]
  void* out;                   // [T, H * Dv]
  const int* cu_seqlens;
  const int* seq_slots;
  int H, D, Dv;
};

template <typename T>
__global__ void __launch_bounds__(ML_THREADS) mlstm_walk_kernel(MlArgs a) {
  extern __shared__ float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H;
  float* S = sm;                     // D * Dv
  float* nn = S + D * Dv;            // D
  float* q = nn + D;                 // D
  float* k = q + D;                  // D
  float* v = k + D;                  // Dv
  float* part = v + Dv;              // slices * Dv
  float* o = part + (ML_THREADS / 32) * Dv;   // Dv
  __shared__ float red[33];
  __shared__ float sc[4];
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
  const int t0 = a.cu_seqlens[s], t1 = a.cu_seqlens[s + 1];
  const int slot = a.seq_slots[s];
  float* Sg = a.S + ((size_t)slot * H + h) * D * Dv;
  float* ng = a.n + ((size_t)slot * H + h) * D;
  float* mg = a.m + (size_t)slot * H + h;
  for (int i = tid; i < D * Dv; i += ML_THREADS) S[i] = Sg[i];
  for (int i = tid; i < D; i += ML_THREADS) nn[i] = ng[i];
  float m = *mg;
  const T* proj = (const T*)a.proj;
  T* out = (T*)a.out;
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int NW = ML_THREADS / 32;
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const T* pr = proj + (size_t)t * a.row;
    for (int i = tid; i < D; i += ML_THREADS) {
      q[i] = to_f32(pr[a.q_off + h * D + i]) * a.q_scale;
      k[i] = to_f32(pr[a.k_off + h * D + i]);
    }
    for (int i = tid; i < Dv; i += ML_THREADS) v[i] = to_f32(pr[a.v_off + h * Dv + i]);
    const float gi = ml_cap(a.gates[(size_t)t * 2 * H + h] + a.bias[h], a.cap);
    const float gf = ml_logsigmoid(ml_cap(a.gates[(size_t)t * 2 * H + H + h] + a.bias[H + h], a.cap));
    const float m_new = fmaxf(gf + m, gi);
    const float fa = expf(gf + m - m_new), fb = expf(gi - m_new);
    m = m_new;
    __syncthreads();
    // the state's rows d = warp, warp + NW, ...: update, and this warp's share of S^T q per column
    for (int c0 = 0; c0 < Dv; c0 += 32) {
      const int c = c0 + lane;
      float acc = 0.f;
      if (c < Dv) {
        const float vc = v[c];
        for (int d = warp; d < D; d += NW) {
          const float x = fa * S[d * Dv + c] + fb * k[d] * vc;
          S[d * Dv + c] = x;
          acc = fmaf(x, q[d], acc);
        }
        part[warp * Dv + c] = acc;
      }
    }
    float nq = 0.f;
    for (int d = tid; d < D; d += ML_THREADS) {
      const float x = fa * nn[d] + fb * k[d];
      nn[d] = x;
      nq = fmaf(x, q[d], nq);
    }
    nq = block_sum(nq, red);               // also orders part[] before the reads below
    const float den = fmaxf(fabsf(nq), expf(-m)) + a.den_eps;
    float ss = 0.f;
    for (int c = tid; c < Dv; c += ML_THREADS) {
      float num = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) num += part[w * Dv + c];
      const float x = num / den;
      o[c] = x;
      ss += x * x;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)Dv + a.eps);
    for (int c = tid; c < Dv; c += ML_THREADS) {
      const float g = to_f32(pr[a.g_off + h * Dv + c]);
      out[(size_t)t * H * Dv + h * Dv + c] = from_f32<T>(o[c] * inv * a.gain[h * Dv + c] * ml_sigmoid(g));
    }
    __syncthreads();
  }
  for (int i = tid; i < D * Dv; i += ML_THREADS) Sg[i] = S[i];
  for (int i = tid; i < D; i += ML_THREADS) ng[i] = nn[i];
  if (tid == 0) *mg = m;
  (void)sc;
}

static size_t ml_walk_smem(int D, int Dv) {
  return (size_t)(D * Dv + 3 * D + Dv + (ML_THREADS / 32) * Dv + Dv) * sizeof(float);
}

extern "C" int sx_mlstm_walk_fits(int D, int Dv) { return ml_walk_smem(D, Dv) <= 200 * 1024 ? 1 : 0; }

extern "C" int sx_mlstm(const void* proj, int row, int q_off, int k_off, int v_off, int g_off, const float* gates,
                        const float* bias, float cap, float q_scale, const float* gain, float eps, float den_eps,
                        float* S, float* n, float* m, void* out, const int* cu_seqlens, const int* seq_slots,
                        int n_seqs, int H, int D, int Dv, int dt, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || D <= 0 || Dv <= 0 || H > 65535 || n_seqs > 65535) return SX_ERR_SIZE;
  const size_t smem = ml_walk_smem(D, Dv);
  if (smem > 200 * 1024) return SX_ERR_SIZE;
  MlArgs a = {proj, row, q_off, k_off, v_off, g_off, gates, bias, cap, q_scale, eps, den_eps, gain, S, n, m, out,
              cu_seqlens, seq_slots, H, D, Dv};
  if (dt == SX_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_walk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(mlstm_walk_kernel<float>, dim3(H, n_seqs), dim3(ML_THREADS), smem, stream, a);
  }
  if (dt == SX_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_walk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(mlstm_walk_kernel<bf16>, dim3(H, n_seqs), dim3(ML_THREADS), smem, stream, a);
  }
  return SX_ERR_DTYPE;
}
