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
//   mlstm_gates_kernel  a block a (piece, head, sequence): the gates of its tokens, the running sums b of f inside the
//                       piece and the piece's own maximum m_loc = max_j (b_end - b_j + i_j).
//   mlstm_piece_kernel  a block a (piece, head, sequence): U = sum_j exp(b_end - b_j + i_j - m_loc) k_j v_j^T and the
//                       same sum of k_j alone.
//   mlstm_carry_kernel  a block a (head, sequence) and slice of the state: the maximum at every piece's begin
//                       (m_end = max(b_end + m_begin, m_loc)) and the state there,
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

// in_place: the matrix is too large for shared memory and is updated where it lies (every element is read and written
// by one thread only)
template <typename T>
__global__ void __launch_bounds__(ML_THREADS) mlstm_walk_kernel(MlArgs a, int in_place) {
  extern __shared__ float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H;
  float* S = sm;                     // D * Dv (not with in_place)
  float* nn = in_place ? sm : S + D * Dv;            // D
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
  if (in_place) S = Sg;
  else
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
  if (!in_place)
    for (int i = tid; i < D * Dv; i += ML_THREADS) Sg[i] = S[i];
  for (int i = tid; i < D; i += ML_THREADS) ng[i] = nn[i];
  if (tid == 0) *mg = m;
  (void)sc;
}

static size_t ml_walk_smem(int D, int Dv, bool in_place = false) {
  return (size_t)((in_place ? 0 : D * Dv) + 3 * D + Dv + (ML_THREADS / 32) * Dv + Dv) * sizeof(float);
}

extern "C" int sx_mlstm_walk_fits(int D, int Dv) { return ml_walk_smem(D, Dv) <= 200 * 1024 ? 1 : 0; }

// ---------------------------------------------------------------------------------------------------------------
// pieces of ML_PIECE tokens.  Scratch: tok [T, H, 2] = (a_j = i_j - b_j, b_j) with b the running sum of f inside the
// piece; info [S, P, H, 4] = (b_end, m_loc, m_begin, m_end); st [S, P, H, D * Dv + D]: first each piece's own sums
// (U, then the sum of k alone), which the carry kernel replaces by the state at the piece's begin.
// ---------------------------------------------------------------------------------------------------------------
struct MlPieces {
  float* tok;
  float* info;
  float* st;
  int P;
};

// a block a (piece, head, sequence): the piece's gates, running sums and own maximum (info[0], info[1])
__global__ void __launch_bounds__(ML_PIECE) mlstm_gates_kernel(MlArgs a, MlPieces w) {
  __shared__ float gf[ML_PIECE], av[ML_PIECE];
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x, h = blockIdx.y, s = blockIdx.z, j = threadIdx.x, H = a.H;
  const int t0 = a.cu_seqlens[s] + p * ML_PIECE, len = a.cu_seqlens[s + 1] - t0;
  if (len <= 0) return;
  const int L = min(ML_PIECE, len);
  const int t = t0 + j;
  float gi = 0.f;
  if (j < L) {
    gi = ml_cap(a.gates[(size_t)t * 2 * H + h] + a.bias[h], a.cap);
    gf[j] = ml_logsigmoid(ml_cap(a.gates[(size_t)t * 2 * H + H + h] + a.bias[H + h], a.cap));
  }
  __syncthreads();
  float b = 0.f;
  if (j < L) {
    for (int x = 0; x <= j; ++x) b += gf[x];
    av[j] = gi - b;
    w.tok[((size_t)t * H + h) * 2] = gi - b;
    w.tok[((size_t)t * H + h) * 2 + 1] = b;
  }
  __syncthreads();
  if (j == L - 1) {                    // b is b_end here
    float mloc = -INFINITY;
    for (int x = 0; x < L; ++x) mloc = fmaxf(mloc, b + av[x]);
    float* o = w.info + (((size_t)s * w.P + p) * H + h) * 4;
    o[0] = b; o[1] = mloc;
  }
}

// U = sum_j w_j k_j v_j^T (D x Dv) and sum_j w_j k_j (D), w_j = exp(a_j + b_end - m_loc); 4 x 4 results a thread
template <typename T>
__global__ void __launch_bounds__(ML_THREADS) mlstm_piece_kernel(MlArgs a, MlPieces w) {
  extern __shared__ float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H;
  float* ks = sm;                    // ML_PIECE * D, already times w_j
  float* vs = ks + ML_PIECE * D;     // ML_PIECE * Dv
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x, h = blockIdx.y, s = blockIdx.z, tid = threadIdx.x;
  const int t0 = a.cu_seqlens[s] + p * ML_PIECE, len = a.cu_seqlens[s + 1] - t0;
  if (len <= 0) return;
  const int L = min(ML_PIECE, len);
  const float* info = w.info + (((size_t)s * w.P + p) * H + h) * 4;
  const float shift = info[0] - info[1];
  const T* proj = (const T*)a.proj;
  for (int i = tid; i < L * D; i += ML_THREADS) {
    const int j = i / D, d = i % D;
    const float wj = expf(w.tok[((size_t)(t0 + j) * H + h) * 2] + shift);
    ks[i] = to_f32(proj[(size_t)(t0 + j) * a.row + a.k_off + h * D + d]) * wj;
  }
  for (int i = tid; i < L * Dv; i += ML_THREADS) {
    const int j = i / Dv, c = i % Dv;
    vs[i] = to_f32(proj[(size_t)(t0 + j) * a.row + a.v_off + h * Dv + c]);
  }
  __syncthreads();
  float* st = w.st + (((size_t)s * w.P + p) * H + h) * ((size_t)D * Dv + D);
  const int tilesV = (Dv + 63) / 64, tilesD = (D + 15) / 16;       // a tile: 16 rows d x 64 columns, 4 x 1... see below
  // thread (ty, tx) of a 16 x 16 grid owns rows d = 4 ty .. 4 ty + 3 (of a 64-row tile) and columns c = tx + 16 x
  const int tx = tid & 15, ty = tid >> 4;
  (void)tilesV; (void)tilesD;
  for (int d0 = 0; d0 < D; d0 += 64)
    for (int c0 = 0; c0 < Dv; c0 += 64) {
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[i][x] = 0.f;
      for (int j = 0; j < L; ++j) {
        float kk[4], vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const int d = d0 + ty * 4 + i; kk[i] = d < D ? ks[j * D + d] : 0.f; }
#pragma unroll
        for (int x = 0; x < 4; ++x) { const int c = c0 + tx + 16 * x; vv[x] = c < Dv ? vs[j * Dv + c] : 0.f; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int x = 0; x < 4; ++x) acc[i][x] = fmaf(kk[i], vv[x], acc[i][x]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = d0 + ty * 4 + i;
        if (d >= D) continue;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int c = c0 + tx + 16 * x;
          if (c < Dv) st[(size_t)d * Dv + c] = acc[i][x];
        }
      }
    }
  for (int d = tid; d < D; d += ML_THREADS) {
    float acc = 0.f;
    for (int j = 0; j < L; ++j) acc += ks[j * D + d];
    st[(size_t)D * Dv + d] = acc;
  }
}

// every thread walks the pieces' maxima itself (m_end = max(b_end + m_begin, m_loc), a few numbers a piece) and one
// thread a (head, sequence) leaves them for the apply kernel (info[2], info[3]); the sequence's new maximum is written
// by the apply kernel, after every block here has read the old one
__global__ void __launch_bounds__(ML_THREADS) mlstm_carry_kernel(MlArgs a, MlPieces w) {
  pdl_wait();
  pdl_trigger();
  const int H = a.H, h = blockIdx.y, s = blockIdx.z;
  const size_t n_el = (size_t)a.D * a.Dv + a.D;
  const size_t e = (size_t)blockIdx.x * ML_THREADS + threadIdx.x;
  if (e >= n_el) return;
  const int len = a.cu_seqlens[s + 1] - a.cu_seqlens[s];
  const int np = (len + ML_PIECE - 1) / ML_PIECE;
  const int slot = a.seq_slots[s];
  float* home = e < (size_t)a.D * a.Dv ? a.S + ((size_t)slot * H + h) * a.D * a.Dv + e
                                        : a.n + ((size_t)slot * H + h) * a.D + (e - (size_t)a.D * a.Dv);
  float S = *home;
  float m = a.m[(size_t)slot * H + h];
  for (int p0 = 0; p0 < np; p0 += 8) {
    float own[8], bend[8], mloc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (p0 + i < np) {                 // eight pieces' loads on the way before the chain below waits for any
        const float* info = w.info + (((size_t)s * w.P + p0 + i) * H + h) * 4;
        bend[i] = info[0]; mloc[i] = info[1];
        own[i] = w.st[(((size_t)s * w.P + p0 + i) * H + h) * n_el + e];
      }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (p0 + i < np) {
        const float mend = fmaxf(bend[i] + m, mloc[i]);
        const float fa = expf(bend[i] + m - mend), fb = expf(mloc[i] - mend);
        if (e == 0) {
          float* info = w.info + (((size_t)s * w.P + p0 + i) * H + h) * 4;
          info[2] = m; info[3] = mend;
        }
        w.st[(((size_t)s * w.P + p0 + i) * H + h) * n_el + e] = S;
        S = fa * S + fb * own[i];
        m = mend;
      }
  }
  *home = S;
}

// CV: columns of the result a thread owns (Dv <= 16 * CV)
template <typename T, int CV>
__global__ void __launch_bounds__(ML_THREADS) mlstm_apply_kernel(MlArgs a, MlPieces w) {
  extern __shared__ float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H, DS = D + 1;
  float* qs = sm;                        // ML_PIECE * DS
  float* ks = qs + ML_PIECE * DS;        // ML_PIECE * DS
  float* vs = ks + ML_PIECE * DS;        // ML_PIECE * Dv
  // the weighted scores, ML_PIECE * (ML_PIECE + 1): in the keys' place once the scores are made (the keys are not read
  // again), where that is large enough: two blocks then fit an SM at head sizes of 128
  const bool ps_over_keys = D >= ML_PIECE;
  float* ps = ps_over_keys ? ks : vs + ML_PIECE * Dv;
  float* av = vs + ML_PIECE * Dv + (ps_over_keys ? 0 : ML_PIECE * (ML_PIECE + 1));   // a_j
  float* bv = av + ML_PIECE;             // b_i
  float* Mv = bv + ML_PIECE;             // M_i = max(m_begin, max_{j<=i} a_j)
  float* dn = Mv + ML_PIECE;             // denominators
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x, h = blockIdx.y, s = blockIdx.z, tid = threadIdx.x;
  const int t0 = a.cu_seqlens[s] + p * ML_PIECE, len = a.cu_seqlens[s + 1] - t0;
  if (len <= 0) return;
  const int L = min(ML_PIECE, len);
  const float* info = w.info + (((size_t)s * w.P + p) * H + h) * 4;
  const float mbeg = info[2];
  if (tid == 0 && len <= ML_PIECE) a.m[(size_t)a.seq_slots[s] * H + h] = info[3];     // the last piece: the new maximum
  const float* S0 = w.st + (((size_t)s * w.P + p) * H + h) * ((size_t)D * Dv + D);
  const float* n0 = S0 + (size_t)D * Dv;
  const T* proj = (const T*)a.proj;
  for (int i = tid; i < ML_PIECE * D; i += ML_THREADS) {
    const int j = i / D, d = i % D;
    const bool ok = j < L;
    qs[j * DS + d] = ok ? to_f32(proj[(size_t)(t0 + j) * a.row + a.q_off + h * D + d]) * a.q_scale : 0.f;
    ks[j * DS + d] = ok ? to_f32(proj[(size_t)(t0 + j) * a.row + a.k_off + h * D + d]) : 0.f;
  }
  for (int i = tid; i < ML_PIECE * Dv; i += ML_THREADS) {
    const int j = i / Dv, c = i % Dv;
    vs[i] = j < L ? to_f32(proj[(size_t)(t0 + j) * a.row + a.v_off + h * Dv + c]) : 0.f;
  }
  if (tid < ML_PIECE) {
    av[tid] = tid < L ? w.tok[((size_t)(t0 + tid) * H + h) * 2] : -INFINITY;
    bv[tid] = tid < L ? w.tok[((size_t)(t0 + tid) * H + h) * 2 + 1] : 0.f;
  }
  __syncthreads();
  if (tid < ML_PIECE) {
    float M = mbeg;
    for (int j = 0; j <= tid; ++j) M = fmaxf(M, av[j]);
    Mv[tid] = M;
  }
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  {   // scores: rows i = 4 ty + ii, columns j = tx + 16 x; weighted and masked
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[i][x] = 0.f;
#pragma unroll 4
    for (int d = 0; d < D; ++d) {
      float qq[4], kk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qq[i] = qs[(ty * 4 + i) * DS + d];
#pragma unroll
      for (int x = 0; x < 4; ++x) kk[x] = ks[(tx + 16 * x) * DS + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[i][x] = fmaf(qq[i], kk[x], acc[i][x]);
    }
    __syncthreads();             // every thread has read the keys
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int j = tx + 16 * x;
        ps[r * (ML_PIECE + 1) + j] = (j <= r && r < L) ? acc[i][x] * expf(av[j] - Mv[r]) : 0.f;
      }
    }
  }
  __syncthreads();
  if (tid < ML_PIECE) {        // the denominator of row tid
    const int r = tid;
    float nq = 0.f;
    for (int j = 0; j <= r; ++j) nq += ps[r * (ML_PIECE + 1) + j];
    float n0q = 0.f;
    for (int d = 0; d < D; ++d) n0q = fmaf(n0[d], qs[r * DS + d], n0q);
    nq = fmaf(expf(mbeg - Mv[r]), n0q, nq);
    dn[r] = fmaxf(fabsf(nq), expf(-(bv[r] + Mv[r]))) + a.den_eps;
  }
  float acc[4][CV];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int x = 0; x < CV; ++x) acc[i][x] = 0.f;
  // the state at the piece's begin: sum_d q_i[d] S0[d][c], then times exp(m_begin - M_i)
#pragma unroll 4
  for (int d = 0; d < D; ++d) {
    float qq[4], sv[CV];
#pragma unroll
    for (int i = 0; i < 4; ++i) qq[i] = qs[(ty * 4 + i) * DS + d];
#pragma unroll
    for (int x = 0; x < CV; ++x) { const int c = tx + 16 * x; sv[x] = c < Dv ? S0[(size_t)d * Dv + c] : 0.f; }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int x = 0; x < CV; ++x) acc[i][x] = fmaf(qq[i], sv[x], acc[i][x]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float f = expf(mbeg - Mv[ty * 4 + i]);
#pragma unroll
    for (int x = 0; x < CV; ++x) acc[i][x] *= f;
  }
  const int jmax = min(L, ty * 4 + 4);
#pragma unroll 4
  for (int j = 0; j < jmax; ++j) {
    float pp[4], vv[CV];
#pragma unroll
    for (int i = 0; i < 4; ++i) pp[i] = ps[(ty * 4 + i) * (ML_PIECE + 1) + j];
#pragma unroll
    for (int x = 0; x < CV; ++x) { const int c = tx + 16 * x; vv[x] = c < Dv ? vs[j * Dv + c] : 0.f; }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int x = 0; x < CV; ++x) acc[i][x] = fmaf(pp[i], vv[x], acc[i][x]);
  }
  __syncthreads();             // dn[] is written
  T* out = (T*)a.out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    const float inv_den = 1.f / dn[r];
    float ss = 0.f;
#pragma unroll
    for (int x = 0; x < CV; ++x) { acc[i][x] *= inv_den; ss += acc[i][x] * acc[i][x]; }   // columns beyond Dv hold 0
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);            // the 16 threads of a row
    const float inv = rsqrtf(ss / (float)Dv + a.eps);
    if (r < L) {
      const size_t t = (size_t)(t0 + r);
#pragma unroll
      for (int x = 0; x < CV; ++x) {
        const int c = tx + 16 * x;
        if (c < Dv) {
          const float g = to_f32(proj[t * a.row + a.g_off + h * Dv + c]);
          out[t * H * Dv + h * Dv + c] = from_f32<T>(acc[i][x] * inv * a.gain[h * Dv + c] * ml_sigmoid(g));
        }
      }
    }
  }
}

static size_t ml_piece_smem(int D, int Dv) { return (size_t)ML_PIECE * (D + Dv) * sizeof(float); }
static size_t ml_apply_smem(int D, int Dv) {
  return (size_t)(2 * ML_PIECE * (D + 1) + ML_PIECE * Dv + (D >= ML_PIECE ? 0 : ML_PIECE * (ML_PIECE + 1)) + 4 * ML_PIECE) * sizeof(float);
}

extern "C" int sx_mlstm_piece_tokens() { return ML_PIECE; }
extern "C" int sx_mlstm_pieces_fit(int D, int Dv) {
  return (Dv <= 256 && ml_apply_smem(D, Dv) <= 200 * 1024 && ml_piece_smem(D, Dv) <= 200 * 1024) ? 1 : 0;
}

template <typename T>
static int mlstm_pieces_launch(MlArgs a, MlPieces w, int n_seqs, cudaStream_t stream) {
  const int H = a.H, D = a.D, Dv = a.Dv;
  int rc = sx_launch(mlstm_gates_kernel, dim3(w.P, H, n_seqs), dim3(ML_PIECE), 0, stream, a, w);
  if (rc) return rc;
  const size_t sp = ml_piece_smem(D, Dv), sa = ml_apply_smem(D, Dv);
  if (sp > 48 * 1024) cudaFuncSetAttribute(mlstm_piece_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sp);
  rc = sx_launch(mlstm_piece_kernel<T>, dim3(w.P, H, n_seqs), dim3(ML_THREADS), sp, stream, a, w);
  if (rc) return rc;
  const size_t n_el = (size_t)D * Dv + D;
  rc = sx_launch(mlstm_carry_kernel, dim3((unsigned)((n_el + ML_THREADS - 1) / ML_THREADS), H, n_seqs), dim3(ML_THREADS), 0, stream, a, w);
  if (rc) return rc;
#define ML_APPLY(CV)                                                                                                          \
  do {                                                                                                                        \
    if (sa > 48 * 1024) cudaFuncSetAttribute(mlstm_apply_kernel<T, CV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sa); \
    return sx_launch(mlstm_apply_kernel<T, CV>, dim3(w.P, H, n_seqs), dim3(ML_THREADS), sa, stream, a, w);                    \
  } while (0)
  if (Dv <= 64) ML_APPLY(4);
  if (Dv <= 128) ML_APPLY(8);
  ML_APPLY(16);
#undef ML_APPLY
}

extern "C" int sx_mlstm(const void* proj, int row, int q_off, int k_off, int v_off, int g_off, const float* gates,
                        const float* bias, float cap, float q_scale, const float* gain, float eps, float den_eps,
                        float* S, float* n, float* m, void* out, const int* cu_seqlens, const int* seq_slots,
                        int n_seqs, int H, int D, int Dv, int dt, float* tok, float* info, float* st, int pieces,
                        cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || D <= 0 || Dv <= 0 || H > 65535 || n_seqs > 65535) return SX_ERR_SIZE;
  if (pieces > 0) {         // long portions: pieces of ML_PIECE tokens (the caller has asked sx_mlstm_pieces_fit)
    if (!sx_mlstm_pieces_fit(D, Dv) || tok == nullptr || info == nullptr || st == nullptr) return SX_ERR_SIZE;
    MlArgs a = {proj, row, q_off, k_off, v_off, g_off, gates, bias, cap, q_scale, eps, den_eps, gain, S, n, m, out,
                cu_seqlens, seq_slots, H, D, Dv};
    MlPieces w = {tok, info, st, pieces};
    if (dt == SX_F32) return mlstm_pieces_launch<float>(a, w, n_seqs, stream);
    if (dt == SX_BF16) return mlstm_pieces_launch<bf16>(a, w, n_seqs, stream);
    return SX_ERR_DTYPE;
  }
  const int in_place = ml_walk_smem(D, Dv) > 200 * 1024 ? 1 : 0;
  const size_t smem = ml_walk_smem(D, Dv, in_place != 0);
  if (smem > 200 * 1024) return SX_ERR_SIZE;
  MlArgs a = {proj, row, q_off, k_off, v_off, g_off, gates, bias, cap, q_scale, eps, den_eps, gain, S, n, m, out,
              cu_seqlens, seq_slots, H, D, Dv};
  if (dt == SX_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_walk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(mlstm_walk_kernel<float>, dim3(H, n_seqs), dim3(ML_THREADS), smem, stream, a, in_place);
  }
  if (dt == SX_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_walk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(mlstm_walk_kernel<bf16>, dim3(H, n_seqs), dim3(ML_THREADS), smem, stream, a, in_place);
  }
  return SX_ERR_DTYPE;
}
