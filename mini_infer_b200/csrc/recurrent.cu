// Mixers that carry a state of fixed size from token to token instead of keys and values.
//
// Every request of a step brings q_len[b] consecutive tokens (rows q_start[b] .. of the packed
// activations) and owns row state_slot[b] of a state arena (fp32, zeroed when the request is
// admitted).  All recurrences run in fp32, token by token in the order of the positions, so a
// result never depends on how a prompt was cut into steps or on what else is in the batch (the
// chunked walk of long bfloat16 portions folds whole chunks first, which moves the fp32 rounding).
//
//   mi_causal_conv     per channel: out[t] = b + sum_j w[j] * in[t - (taps-1-j)], in = x + x_bias,
//                      with the taps-1 inputs before the portion taken from the state (zeros before
//                      the start of a sequence); optionally SiLU of the result.  Does not change the state.
//   mi_rglru_scan      the real-gated linear recurrent unit:
//                        r = sigmoid(gr + br), i = sigmoid(gi + bi), log a = -c * r * softplus(lam),
//                        S = a S + sqrt(1 - a^2) * i * u;   out = T(S * gelu_tanh(y + by))
//                      and, for the convolution in front of it, the new last taps-1 inputs.
//   mi_gla_scan        gated linear attention, per head: S = diag(alpha) S + k v^T, o = S^T (q * qscale),
//                      alpha = sigmoid(z + bz)^(1/tau), or one fixed decay per head (head_decay).
//                      Optionally the decay and a factor on k come per token and head from a table
//                      (tok_gates), and one more value column of ones rides along (extra_col): the
//                      state then holds sum(k) beside sum(k v^T), a normaliser.
//   mi_mlstm_gates     the scalar gates of a matrix memory with a running maximum, per head and token:
//                        i = cap tanh((zi + bi) / cap), f = logsigmoid(cap tanh((zf + bf) / cap)),
//                        m' = max(f + m, i);  gates = (exp(f + m - m'), exp(i - m'), m');  m <- m'
//   mi_delta_scan      the gated delta rule with a decay per key channel, per head:
//                        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                      with q and k made unit vectors per head first (q also times q_scale),
//                      g = exp(-exp(A_log) * softplus(z + dt_bias)), beta = sigmoid(b); and, for the
//                      convolution in front of it, the new last taps-1 inputs.
//   mi_headnorm_gate   out = T(o / sqrt(mean_head(o^2) + eps) * w * act(g) * scale) per head of dv.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define MAX_TAPS 16

// ------------------------------------------------------------------------------------------
// causal convolution over a portion, with the state's tail in front of it
// state row of a request: [taps-1][C] inputs (oldest first), then whatever else the mixer keeps
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ x_bias,
                                   const float* __restrict__ w, const float* __restrict__ b,
                                   const float* __restrict__ state, long long state_stride,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ state_slot, T* __restrict__ out, int out_stride,
                                   int C, int taps, int tile, int act) {
  mi_pdl_enter();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.z;
  const int len = q_len[req];
  const int t0 = blockIdx.y * tile;
  if (c >= C || t0 >= len) return;
  const int row0 = q_start[req];
  const float* tail = state + (size_t)state_slot[req] * state_stride;
  float wv[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) wv[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
  const float xb = x_bias ? x_bias[c] : 0.f, bias = b ? b[c] : 0.f;
  const int t1 = min(len, t0 + tile);
  for (int t = t0; t < t1; ++t) {
    float acc = bias;
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      if (j < taps) {
        const int src = t - (taps - 1 - j);
        const float v = src >= 0 ? mi_to_float(x[(size_t)(row0 + src) * x_stride + c]) + xb
                                 : tail[(size_t)(taps - 1 + src) * C + c];
        acc = fmaf(wv[j], v, acc);
      }
    }
    if (act == 1) acc = acc / (1.f + expf(-acc));   // SiLU
    out[(size_t)(row0 + t) * out_stride + c] = mi_from_float<T>(acc);
  }
}

extern "C" int mi_causal_conv(const void* x, int x_stride, const float* x_bias, const float* w, const float* b,
                              const float* state, long long state_stride, const int* q_start, const int* q_len,
                              const int* state_slot, void* out, int out_stride, int n_requests, int max_q_len,
                              int C, int taps, int act, int dtype, cudaStream_t stream) {
  if (n_requests <= 0 || max_q_len <= 0) return 0;
  if (act != 0 && act != 1) MI_REFUSE("causal_conv: unknown activation %d", act);
  if (taps < 1 || taps > MAX_TAPS) MI_REFUSE("causal_conv: %d taps (1 to %d are taken)", taps, MAX_TAPS);
  const int tile = 16;
  dim3 grid((C + 127) / 128, (max_q_len + tile - 1) / tile, n_requests);
  if (grid.y > 65535 || grid.z > 65535) MI_REFUSE("causal_conv: too many tiles for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((causal_conv_kernel<float>), grid, 128, 0, stream, (const float*)x, x_stride, x_bias, w, b, state,
              state_stride, q_start, q_len, state_slot, (float*)out, out_stride, C, taps, tile, act);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((causal_conv_kernel<bf16>), grid, 128, 0, stream, (const bf16*)x, x_stride, x_bias, w, b, state,
              state_stride, q_start, q_len, state_slot, (bf16*)out, out_stride, C, taps, tile, act);
  else
    MI_REFUSE("causal_conv: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// real-gated linear recurrent unit.  One thread per (request, channel) walks the portion.
// gates [blocks][M][2 * bw]: for block k, row m: the r pre-activations of its bw channels, then the i ones.
// state row: [taps-1][C] convolution inputs, then [C] the recurrent state.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float mi_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float mi_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float mi_gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ gates, int M, int bw,
                                  const float* __restrict__ br, const float* __restrict__ bi,
                                  const float* __restrict__ lam, float decay_scale,
                                  const T* __restrict__ u, int u_stride,
                                  const T* __restrict__ y, int y_stride, const float* __restrict__ y_bias,
                                  const T* __restrict__ xin, int xin_stride, const float* __restrict__ xin_bias,
                                  float* __restrict__ state, long long state_stride, int taps,
                                  const int* __restrict__ q_start, const int* __restrict__ q_len,
                                  const int* __restrict__ state_slot, T* __restrict__ out, int out_stride, int C) {
  mi_pdl_enter();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.y;
  if (c >= C) return;
  const int len = q_len[req], row0 = q_start[req];
  float* st = state + (size_t)state_slot[req] * state_stride;
  float* Sp = st + (size_t)(taps - 1) * C + c;
  float S = *Sp;
  const int blk = c / bw, cj = c - blk * bw;
  const float* g = gates + ((size_t)blk * M + row0) * (2 * bw) + cj;
  const float vbr = br[c], vbi = bi[c], yb = y_bias ? y_bias[c] : 0.f;
  const float sp = decay_scale * mi_softplus(lam[c]);
  for (int t = 0; t < len; ++t) {
    const float r = mi_sigmoid(g[0] + vbr), ig = mi_sigmoid(g[bw] + vbi);
    g += 2 * bw;
    const float log_a = -sp * r;
    const float a = expf(log_a);
    const float mult = sqrtf(-expm1f(2.f * log_a));
    const float uv = mi_to_float(u[(size_t)(row0 + t) * u_stride + c]);
    S = fmaf(a, S, mult * (ig * uv));
    const float yv = mi_gelu_tanh(mi_to_float(y[(size_t)(row0 + t) * y_stride + c]) + yb);
    out[(size_t)(row0 + t) * out_stride + c] = mi_from_float<T>(S * yv);
  }
  *Sp = S;
  // the convolution's next tail: the last taps-1 of (old tail, this portion's inputs)
  if (taps > 1) {
    const float xb = xin_bias ? xin_bias[c] : 0.f;
    float keep[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
      if (j < taps - 1) {
        const int src = len - (taps - 1) + j;   // portion offset of the j-th kept input
        keep[j] = src >= 0 ? mi_to_float(xin[(size_t)(row0 + src) * xin_stride + c]) + xb
                           : st[(size_t)(taps - 1 + src) * C + c];
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
  }
}

extern "C" int mi_rglru_scan(const float* gates, int M, int bw, const float* br, const float* bi, const float* lam,
                             float decay_scale, const void* u, int u_stride, const void* y, int y_stride,
                             const float* y_bias, const void* xin, int xin_stride, const float* xin_bias,
                             float* state, long long state_stride, int taps, const int* q_start, const int* q_len,
                             const int* state_slot, void* out, int out_stride, int n_requests, int C, int dtype,
                             cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) MI_REFUSE("rglru: %d taps (1 to %d are taken)", taps, MAX_TAPS);
  if (bw <= 0 || C % bw) MI_REFUSE("rglru: %d channels are no whole number of blocks of %d", C, bw);
  if (n_requests > 65535) MI_REFUSE("rglru: too many requests for one launch");
  const int threads = C >= 2048 ? 64 : 32;   // many small blocks: the walk is latency-bound
  dim3 grid((C + threads - 1) / threads, n_requests);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((rglru_scan_kernel<float>), grid, threads, 0, stream, gates, M, bw, br, bi, lam, decay_scale,
              (const float*)u, u_stride, (const float*)y, y_stride, y_bias, (const float*)xin, xin_stride, xin_bias,
              state, state_stride, taps, q_start, q_len, state_slot, (float*)out, out_stride, C);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((rglru_scan_kernel<bf16>), grid, threads, 0, stream, gates, M, bw, br, bi, lam, decay_scale,
              (const bf16*)u, u_stride, (const bf16*)y, y_stride, y_bias, (const bf16*)xin, xin_stride, xin_bias,
              state, state_stride, taps, q_start, q_len, state_slot, (bf16*)out, out_stride, C);
  else
    MI_REFUSE("rglru: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// The same recurrence for long portions, cut into chunks of `chunk` tokens that run side by side.
// Pass 1: every (request, chunk, channel) folds its chunk into S_end = A * S_begin + B.  Pass 2: it
// walks the chunks before its own to get S_begin (from the state as pass 1 saved it), then its own
// tokens exactly as the walk above does.  The last chunk stores the state and the convolution's tail.
// scratch: [requests][max_chunks][2][C] chunk summaries, then [requests][C] the states at the start.
// ------------------------------------------------------------------------------------------
struct RglruTerms { float a, b; };

template <typename T>
__device__ __forceinline__ RglruTerms rglru_terms(const float* g, int bw, float vbr, float vbi, float sp, const T* u,
                                                  size_t row, int u_stride, int c) {
  const float r = mi_sigmoid(g[0] + vbr), ig = mi_sigmoid(g[bw] + vbi);
  const float log_a = -sp * r;
  RglruTerms t;
  t.a = expf(log_a);
  t.b = sqrtf(-expm1f(2.f * log_a)) * (ig * mi_to_float(u[row * u_stride + c]));
  return t;
}

template <typename T, int PASS>
__global__ void rglru_chunk_kernel(const float* __restrict__ gates, int M, int bw,
                                   const float* __restrict__ br, const float* __restrict__ bi,
                                   const float* __restrict__ lam, float decay_scale,
                                   const T* __restrict__ u, int u_stride,
                                   const T* __restrict__ y, int y_stride, const float* __restrict__ y_bias,
                                   const T* __restrict__ xin, int xin_stride, const float* __restrict__ xin_bias,
                                   float* __restrict__ state, long long state_stride, int taps,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ state_slot, T* __restrict__ out, int out_stride, int C,
                                   float* __restrict__ scratch, int max_chunks, int chunk, int n_requests) {
  mi_pdl_enter();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int ci = blockIdx.y, req = blockIdx.z;
  if (c >= C) return;
  const int len = q_len[req], row0 = q_start[req];
  const int t0 = ci * chunk;
  if (t0 >= len) return;
  const int t1 = min(len, t0 + chunk);
  float* st = state + (size_t)state_slot[req] * state_stride;
  float* summ = scratch + ((size_t)req * max_chunks) * 2 * C;
  float* start = scratch + (size_t)n_requests * max_chunks * 2 * C + (size_t)req * C;
  const int blk = c / bw, cj = c - blk * bw;
  const float* g = gates + ((size_t)blk * M + row0 + t0) * (2 * bw) + cj;
  const float vbr = br[c], vbi = bi[c];
  const float sp = decay_scale * mi_softplus(lam[c]);
  if (PASS == 1) {
    float A = 1.f, B = 0.f;
#pragma unroll 4
    for (int t = t0; t < t1; ++t, g += 2 * bw) {
      const RglruTerms k = rglru_terms(g, bw, vbr, vbi, sp, u, (size_t)(row0 + t), u_stride, c);
      B = fmaf(k.a, B, k.b);
      A *= k.a;
    }
    summ[((size_t)ci * 2) * C + c] = A;
    summ[((size_t)ci * 2 + 1) * C + c] = B;
    if (ci == 0) start[c] = st[(size_t)(taps - 1) * C + c];
    return;
  }
  float S = start[c];
  for (int p = 0; p < ci; ++p) S = fmaf(summ[((size_t)p * 2) * C + c], S, summ[((size_t)p * 2 + 1) * C + c]);
  const float yb = y_bias ? y_bias[c] : 0.f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, g += 2 * bw) {
    const RglruTerms k = rglru_terms(g, bw, vbr, vbi, sp, u, (size_t)(row0 + t), u_stride, c);
    S = fmaf(k.a, S, k.b);
    const float yv = mi_gelu_tanh(mi_to_float(y[(size_t)(row0 + t) * y_stride + c]) + yb);
    out[(size_t)(row0 + t) * out_stride + c] = mi_from_float<T>(S * yv);
  }
  if (t1 < len) return;
  st[(size_t)(taps - 1) * C + c] = S;
  if (taps > 1) {
    const float xb = xin_bias ? xin_bias[c] : 0.f;
    float keep[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
      if (j < taps - 1) {
        const int src = len - (taps - 1) + j;
        keep[j] = src >= 0 ? mi_to_float(xin[(size_t)(row0 + src) * xin_stride + c]) + xb
                           : st[(size_t)(taps - 1 + src) * C + c];
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
  }
}

extern "C" long long mi_rglru_chunked_scratch(int n_requests, int max_chunks, int C) {
  return ((long long)n_requests * max_chunks * 2 + n_requests) * C;
}

extern "C" int mi_rglru_scan_chunked(const float* gates, int M, int bw, const float* br, const float* bi,
                                     const float* lam, float decay_scale, const void* u, int u_stride, const void* y,
                                     int y_stride, const float* y_bias, const void* xin, int xin_stride,
                                     const float* xin_bias, float* state, long long state_stride, int taps,
                                     const int* q_start, const int* q_len, const int* state_slot, void* out,
                                     int out_stride, int n_requests, int C, float* scratch, int max_chunks, int chunk,
                                     int dtype, cudaStream_t stream) {
  if (n_requests <= 0 || max_chunks <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) MI_REFUSE("rglru: %d taps (1 to %d are taken)", taps, MAX_TAPS);
  if (bw <= 0 || C % bw) MI_REFUSE("rglru: %d channels are no whole number of blocks of %d", C, bw);
  if (chunk <= 0 || max_chunks > 65535 || n_requests > 65535) MI_REFUSE("rglru: too many chunks or requests for one launch");
  dim3 grid((C + 127) / 128, max_chunks, n_requests);
#define MI_GO(T, PASS)                                                                                               \
  MI_LAUNCH((rglru_chunk_kernel<T, PASS>), grid, 128, 0, stream, gates, M, bw, br, bi, lam, decay_scale, (const T*)u, \
            u_stride, (const T*)y, y_stride, y_bias, (const T*)xin, xin_stride, xin_bias, state, state_stride, taps,   \
            q_start, q_len, state_slot, (T*)out, out_stride, C, scratch, max_chunks, chunk, n_requests)
  if (dtype == MI_DTYPE_F32) {
    MI_GO(float, 1);
    MI_GO(float, 2);
  } else if (dtype == MI_DTYPE_BF16) {
    MI_GO(bf16, 1);
    MI_GO(bf16, 2);
  } else {
    MI_REFUSE("rglru: unknown dtype %d", dtype);
  }
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// gated linear attention.  A block owns 32 value columns of one head of one request; thread
// (tx, ty) keeps rows ty*R .. ty*R+R-1 of column tx of the state in registers.  Tokens are taken in
// groups of GL: q, k, alpha and v of a group are staged in shared memory, every thread walks the
// group updating its rows and leaving its share of each o in shared memory, and the shares are
// added in a fixed order.
// ------------------------------------------------------------------------------------------
#define GLA_R 8
#define GLA_L 16

template <typename TQ, typename T, int MAXT>
__global__ void __launch_bounds__(MAXT) gla_scan_kernel(const TQ* __restrict__ q, const TQ* __restrict__ k, int qk_stride,
                                const T* __restrict__ v, int stride,
                                const float* __restrict__ z, int z_stride, const float* __restrict__ z_bias,
                                float inv_tau, float q_scale, float* __restrict__ state, long long state_stride,
                                const int* __restrict__ q_start, const int* __restrict__ q_len,
                                const int* __restrict__ state_slot, float* __restrict__ o, int o_stride,
                                int heads, int dk, int dv, int pass, int chunk_len, int n_chunks,
                                float* __restrict__ scratch, const float* __restrict__ head_decay,
                                const float* __restrict__ tok_gates, int extra_col) {
  // head_decay [heads]: one fixed decay per head in the place of alpha (z is then not read).
  // tok_gates [M, heads, 3]: per token and head the decay (all key channels alike) and a factor on k
  // (z and head_decay are then not read).  extra_col: the head has dv + 1 value columns, the last one
  // all ones, in the state and in o alike (dv below counts it; v has one column less).
  // q and k may be fp32 rows of their own (what a rotation left in fp32) beside bfloat16 values.
  // pass 0: the whole portion, from and into the state.  Long portions run as chunks side by side:
  // pass 1 folds every chunk into (A, B) with S_end = diag(A) S_begin + B (and saves the state the
  // portion starts from), pass 2 walks the chunks before its own to get S_begin and then its own
  // tokens as pass 0 does; the last chunk stores the state.
  // scratch: per (request, chunk, head) A [dk] and B [dk, dv]; then per (request, head) the state at the start.
  mi_pdl_enter();
  extern __shared__ float sm[];
  const int KP = blockDim.y;
  float* qs = sm;                       // [GLA_L][dk]
  float* ks = qs + GLA_L * dk;          // [GLA_L][dk]
  float* as = ks + GLA_L * dk;          // [GLA_L][dk]
  float* vs = as + GLA_L * dk;          // [GLA_L][32]
  float* part = vs + GLA_L * 32;        // [GLA_L][KP][32]
  const int tx = threadIdx.x, ty = threadIdx.y, tid = ty * 32 + tx, nthreads = KP * 32;
  const int head = blockIdx.y, req = blockIdx.z / n_chunks, chunk = blockIdx.z - req * n_chunks;
  const int j = blockIdx.x * 32 + tx;   // value column
  const int dv_in = dv - extra_col;     // columns that v brings
  const int len_all = q_len[req];
  const int c0 = pass ? chunk * chunk_len : 0;
  if (c0 >= len_all) return;
  const int len = (pass ? min(len_all, c0 + chunk_len) : len_all) - c0, row0 = q_start[req] + c0;
  const bool last = c0 + len == len_all;
  float* S = state + (size_t)state_slot[req] * state_stride + (size_t)head * dk * dv;
  const size_t unit = (size_t)dk + (size_t)dk * dv;
  const int n_req = gridDim.z / n_chunks;
  float* summ = scratch ? scratch + (((size_t)req * n_chunks + chunk) * heads + head) * unit : nullptr;
  float* begin = scratch ? scratch + (size_t)n_req * n_chunks * heads * unit + ((size_t)req * heads + head) * dk * dv
                         : nullptr;
  float s[GLA_R], pa[GLA_R];
#pragma unroll
  for (int i = 0; i < GLA_R; ++i) {
    const int kk = ty * GLA_R + i;
    const bool mine = kk < dk && j < dv;
    pa[i] = 1.f;
    if (pass == 0) {
      s[i] = mine ? S[(size_t)kk * dv + j] : 0.f;
    } else if (pass == 1) {
      s[i] = 0.f;
      if (chunk == 0 && mine) begin[(size_t)kk * dv + j] = S[(size_t)kk * dv + j];
    } else {
      s[i] = mine ? begin[(size_t)kk * dv + j] : 0.f;
      for (int p = 0; p < chunk; ++p) {
        const float* ps = scratch + (((size_t)req * n_chunks + p) * heads + head) * unit;
        if (mine) s[i] = fmaf(ps[kk], s[i], ps[dk + (size_t)kk * dv + j]);
      }
    }
  }
  // A group's q, k, z and v are fetched into registers while the group before is worked on, so that
  // the walk does not stand still for a round trip to memory at every group.
  // Per thread at most 4 elements of each of q, k, z (GLA_L * dk / threads <= 4) and 4 of v (at least
  // 128 threads).
  float pq[4], pk[4], pz[4], pv[4];
  auto fetch = [&](int t0) {
    const int n = min(GLA_L, len - t0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * nthreads;
      if (idx < n * dk) {
        const int l = idx / dk, kk = idx - l * dk;
        const size_t m = (size_t)(row0 + t0 + l);
        pq[i] = mi_to_float(q[m * qk_stride + head * dk + kk]);
        pk[i] = mi_to_float(k[m * qk_stride + head * dk + kk]);
        if (tok_gates) {
          const float* tg = tok_gates + (m * heads + head) * 3;
          pz[i] = tg[0];
          pk[i] *= tg[1];
        } else {
          pz[i] = head_decay ? 0.f : z[m * z_stride + head * dk + kk];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * nthreads;
      if (idx < n * 32) {
        const int l = idx >> 5, jj = blockIdx.x * 32 + (idx & 31);
        pv[i] = jj < dv_in ? mi_to_float(v[(size_t)(row0 + t0 + l) * stride + head * dv_in + jj])
                           : (jj < dv ? 1.f : 0.f);
      }
    }
  };
  if (len > 0) fetch(0);
  for (int t0 = 0; t0 < len; t0 += GLA_L) {
    const int n = min(GLA_L, len - t0);
    __syncthreads();   // the group before is consumed
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * nthreads;
      if (idx < n * dk) {
        const int kk = idx % dk;
        qs[idx] = pq[i] * q_scale;
        ks[idx] = pk[i];
        const float zz = pz[i] + ((z_bias && !tok_gates) ? z_bias[head * dk + kk] : 0.f);
        as[idx] = tok_gates ? pz[i] : head_decay ? head_decay[head]
                             : expf(-mi_softplus(-zz) * inv_tau);     // sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * nthreads;
      if (idx < n * 32) vs[idx] = pv[i];
    }
    __syncthreads();
    if (t0 + GLA_L < len) fetch(t0 + GLA_L);
    for (int l = 0; l < n; ++l) {
      const float vv = vs[l * 32 + tx];
      float po = 0.f;
#pragma unroll
      for (int i = 0; i < GLA_R; ++i) {
        const int kk = ty * GLA_R + i;
        if (kk < dk) {
          const float al = as[l * dk + kk];
          s[i] = fmaf(al, s[i], ks[l * dk + kk] * vv);
          if (pass == 1) pa[i] *= al;
          else po = fmaf(s[i], qs[l * dk + kk], po);
        }
      }
      if (pass != 1) part[(l * KP + ty) * 32 + tx] = po;
    }
    __syncthreads();
    if (pass != 1) for (int l = ty; l < n; l += KP) {
      float sum = 0.f;
      for (int p = 0; p < KP; ++p) sum += part[(l * KP + p) * 32 + tx];
      if (j < dv) o[(size_t)(row0 + t0 + l) * o_stride + head * dv + j] = sum;
    }
  }
#pragma unroll
  for (int i = 0; i < GLA_R; ++i) {
    const int kk = ty * GLA_R + i;
    if (pass == 1) {
      if (kk < dk && j < dv) summ[dk + (size_t)kk * dv + j] = s[i];
      if (kk < dk && j == 0) summ[kk] = pa[i];
      continue;
    }
    if (!last) continue;
    if (kk < dk && j < dv) S[(size_t)kk * dv + j] = s[i];
  }
}

extern "C" long long mi_gla_chunked_scratch(int n_requests, int n_chunks, int heads, int dk, int dv) {
  const long long unit = (long long)dk + (long long)dk * dv;
  return (long long)n_requests * n_chunks * heads * unit + (long long)n_requests * heads * dk * dv;
}

extern "C" int mi_gla_scan(const void* q, const void* k, int qk_stride, int qk_dtype, const void* v, int stride,
                           const float* z, int z_stride,
                           const float* z_bias, float inv_tau, float q_scale, float* state, long long state_stride,
                           const int* q_start, const int* q_len, const int* state_slot, float* o, int o_stride,
                           int n_requests, int heads, int dk, int dv, float* scratch, int n_chunks, int chunk_len,
                           const float* head_decay, const float* tok_gates, int extra_col, int dtype,
                           cudaStream_t stream) {
  // dv counts the value columns of the state and of o; with extra_col v brings one less
  if (n_requests <= 0) return 0;
  if (!z && !head_decay && !tok_gates) MI_REFUSE("gla: neither decays per channel nor per head nor per token");
  if (extra_col != 0 && extra_col != 1) MI_REFUSE("gla: one extra column or none");
  if (dv - extra_col <= 0) MI_REFUSE("gla: no value columns");
  if (n_chunks < 1 || (n_chunks > 1 && (!scratch || chunk_len <= 0))) MI_REFUSE("gla: chunks need scratch memory");
  if ((long long)n_requests * n_chunks > 65535) MI_REFUSE("gla: too many chunks for one launch");
  if (dk <= 0 || dk > 256 || dv <= 0) MI_REFUSE("gla: key size %d must lie in [1, 256], value size %d above 0", dk, dv);
  if (heads > 65535 || n_requests > 65535) MI_REFUSE("gla: too many heads or requests for one launch");
  const int KP = max(4, (dk + GLA_R - 1) / GLA_R);     // at least 128 threads: they also stage the inputs
  dim3 grid((dv + 31) / 32, heads, n_requests * n_chunks), block(32, KP);
  const size_t smem = ((size_t)3 * GLA_L * dk + GLA_L * 32 + (size_t)GLA_L * KP * 32) * sizeof(float);
#define MI_GO(TQ, T)                                                                                      \
  do {                                                                                                    \
    auto kern = KP <= 16 ? gla_scan_kernel<TQ, T, 512> : gla_scan_kernel<TQ, T, 1024>;                    \
    if (smem > 48 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                \
    }                                                                                                     \
    for (int pass = n_chunks > 1 ? 1 : 0; pass <= (n_chunks > 1 ? 2 : 0); ++pass)                         \
      MI_LAUNCH(kern, grid, block, smem, stream, (const TQ*)q, (const TQ*)k, qk_stride, (const T*)v, stride, z, z_stride, \
                z_bias, inv_tau, q_scale, state, state_stride, q_start, q_len, state_slot, o, o_stride, heads, \
                dk, dv, pass, chunk_len, n_chunks, scratch, head_decay, tok_gates, extra_col);              \
  } while (0)
  if (dtype == MI_DTYPE_F32 && qk_dtype == MI_DTYPE_F32) MI_GO(float, float);
  else if (dtype == MI_DTYPE_BF16 && qk_dtype == MI_DTYPE_BF16) MI_GO(bf16, bf16);
  else if (dtype == MI_DTYPE_BF16 && qk_dtype == MI_DTYPE_F32) MI_GO(float, bf16);
  else MI_REFUSE("gla: dtypes %d (q, k) and %d (v) are not taken together", qk_dtype, dtype);
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// scalar gates of a matrix memory with a running maximum.  One block per (request, head) takes the
// portion MLSTM_CHUNK tokens at a time: all threads compute the capped log gates of the chunk's tokens
// into shared memory, one thread walks m' = max(f + m, i) through them in the order of the positions (one
// addition and one maximum per token, the same whatever the cutting), all threads turn (m, m') into the
// decay and the input factor.  A step of single tokens needs one warp per (request, head).
// state row of a request: m [heads] at m_offset.
// ------------------------------------------------------------------------------------------
#define MLSTM_CHUNK 1024
__global__ void mlstm_gates_kernel(const float* __restrict__ zi, const float* __restrict__ zf, int z_stride,
                                   const float* __restrict__ bi, const float* __restrict__ bf_, float cap,
                                   float* __restrict__ state, long long state_stride, long long m_offset,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ state_slot, float* __restrict__ gates, int heads) {
  mi_pdl_enter();
  __shared__ float sh_i[MLSTM_CHUNK], sh_f[MLSTM_CHUNK], sh_m[MLSTM_CHUNK + 1];
  const int req = blockIdx.x / heads, head = blockIdx.x - req * heads;
  const int len = q_len[req], row0 = q_start[req];
  if (len <= 0) return;
  float* mp = state + (size_t)state_slot[req] * state_stride + m_offset + head;
  const float inv_cap = 1.f / cap;
  const float b_i = bi ? bi[head] : 0.f, b_f = bf_ ? bf_[head] : 0.f;
  if (threadIdx.x == 0) sh_m[0] = *mp;
  for (int t0 = 0; t0 < len; t0 += MLSTM_CHUNK) {
    const int n = min(MLSTM_CHUNK, len - t0);
    for (int l = threadIdx.x; l < n; l += blockDim.x) {
      const size_t r = (size_t)(row0 + t0 + l);
      sh_i[l] = cap * tanhf((zi[r * z_stride + head] + b_i) * inv_cap);
      const float a = cap * tanhf((zf[r * z_stride + head] + b_f) * inv_cap);
      sh_f[l] = -mi_softplus(-a);                  // logsigmoid
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // eight tokens' gates into registers, then their eight dependent steps: the loads stay off the chain
      // (a token behind the chunk's end has f = 0, i = -inf and leaves the maximum as it is)
      float run = sh_m[0];
      float f8[8], i8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f8[j] = j < n ? sh_f[j] : 0.f;
        i8[j] = j < n ? sh_i[j] : -INFINITY;
      }
      for (int l = 0; l < n; l += 8) {
        float fn[8], in[8], m8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int k = l + 8 + j;
          fn[j] = k < n ? sh_f[k] : 0.f;
          in[j] = k < n ? sh_i[k] : -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          run = fmaxf(f8[j] + run, i8[j]);
          m8[j] = run;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (l + j < n) sh_m[l + j + 1] = m8[j];
          f8[j] = fn[j];
          i8[j] = in[j];
        }
      }
    }
    __syncthreads();
    for (int l = threadIdx.x; l < n; l += blockDim.x) {
      const float before = sh_m[l], after = sh_m[l + 1];
      float* gp = gates + ((size_t)(row0 + t0 + l) * heads + head) * 3;
      gp[0] = expf(sh_f[l] + before - after);
      gp[1] = expf(sh_i[l] - after);
      gp[2] = after;
    }
    __syncthreads();
    if (threadIdx.x == 0) sh_m[0] = sh_m[n];
  }
  __syncthreads();
  if (threadIdx.x == 0) *mp = sh_m[0];
}

extern "C" int mi_mlstm_gates(const float* zi, const float* zf, int z_stride, const float* bi, const float* bf_,
                              float cap, float* state, long long state_stride, long long m_offset,
                              const int* q_start, const int* q_len, const int* state_slot, float* gates,
                              int n_requests, int heads, int longest, cudaStream_t stream) {
  // longest: the longest portion of the step (sizes the blocks; any value is correct)
  if (n_requests <= 0 || heads <= 0) return 0;
  if (!(cap > 0.f)) MI_REFUSE("mlstm: the gates' cap must be positive, got %g", (double)cap);
  if (m_offset < 0 || m_offset + heads > state_stride) MI_REFUSE("mlstm: the running maxima lie outside the state row");
  if ((long long)n_requests * heads > 0x7fffffffLL) MI_REFUSE("mlstm: too many blocks for one launch");
  const int threads = longest <= 32 ? 32 : (longest <= 256 ? 128 : 512);
  MI_LAUNCH((mlstm_gates_kernel), n_requests * heads, threads, 0, stream, zi, zf, z_stride, bi, bf_, cap, state,
            state_stride, m_offset, q_start, q_len, state_slot, gates, heads);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// gated delta rule.  The columns of a head's state S [dk, dv] evolve independently under the same
// transition.  A warp owns DELTA_NC columns and DELTA_PARTS lanes share a column: lane (part, c) keeps R rows
// of column c in registers, in groups of four consecutive rows dealt out to the parts in turn (group
// part + DELTA_PARTS * i), so that a part reads its q, k and g as 16-byte words that lie side by side with
// the other parts'.  Per token and column: sg = g * s; r = sg . k; p = sg . q; u = beta (v - r);
// s = sg + k u; o = p + u (k . q), which is S^T q after the write.  The two dot products are summed over
// the column's lanes by three exchanges, in an order that depends on nothing but the sizes.  Tokens are staged
// in groups of DELTA_L = DELTA_W, one per warp: the warp makes q and k unit vectors, computes g, beta and k . q,
// and leaves them in shared memory (rows padded to 8 R with k = q = 0, g = 1) for the walk.
// A block has DELTA_W warps, so it owns DELTA_W * DELTA_NC value columns of one head of one request.
// state row of a request: [taps-1][C] convolution inputs (oldest first), then S [heads][dk][dv].
// ------------------------------------------------------------------------------------------
#define DELTA_L 8   // tokens per group: one per warp
#define DELTA_NC 4
#define DELTA_PARTS 8
#define DELTA_W 8
#define DELTA_COLS (DELTA_NC * DELTA_W)

template <typename T, int R>
__global__ void __launch_bounds__(32 * DELTA_W)
delta_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int stride,
                  const float* __restrict__ z, int z_stride, const float* __restrict__ dt_bias,
                  const float* __restrict__ a_log, const T* __restrict__ b, int b_stride, float q_scale,
                  float unit_eps, float* __restrict__ state, long long state_stride, long long s_off,
                  const int* __restrict__ q_start, const int* __restrict__ q_len,
                  const int* __restrict__ state_slot, float* __restrict__ o, int o_stride, int heads, int kv_heads,
                  int dk, int dv, const T* __restrict__ xin, int xin_stride, int C, int taps) {
  mi_pdl_enter();
  constexpr int DKP = DELTA_PARTS * R;   // rows of a staged token, padded
  constexpr int RS = DKP / 32;           // rows a lane stages per token
  constexpr int NG = R / 4;              // groups of four rows per lane
  extern __shared__ __align__(16) float dsm[];
  float* ks = dsm;                       // [DELTA_L][DKP]
  float* qs = ks + DELTA_L * DKP;        // [DELTA_L][DKP]
  float* gs = qs + DELTA_L * DKP;        // [DELTA_L][DKP]
  float* vs = gs + DELTA_L * DKP;        // [DELTA_L][DELTA_COLS]
  float* bs = vs + DELTA_L * DELTA_COLS; // [DELTA_L] beta
  float* kqs = bs + DELTA_L;             // [DELTA_L] k . q
  const int lane = threadIdx.x, warp = threadIdx.y, tid = warp * 32 + lane;
  const int part = lane / DELTA_NC, col = lane % DELTA_NC;
  const int head = blockIdx.y, req = blockIdx.z;
  const int kvh = head / (heads / kv_heads);
  const int len = q_len[req], row0 = q_start[req];
  float* st = state + (size_t)state_slot[req] * state_stride;
  float* S = st + s_off + (size_t)head * dk * dv;
  const int j = blockIdx.x * DELTA_COLS + warp * DELTA_NC + col;   // this lane's column
  const float A = expf(a_log[head]);
  float s[R];
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = 4 * (part + DELTA_PARTS * i) + e;
      s[4 * i + e] = (kk < dk && j < dv) ? S[(size_t)kk * dv + j] : 0.f;
    }
  // Warp w stages token w of a group.  What it needs from global memory (its token's k, q, pre-activations of
  // the decay, beta and the block's values) is fetched into registers one group ahead, before the walk
  // over the group at hand, so that the walk hides the fetch.
  // (kept as loaded: a conversion would wait for the load where it is issued)
  float dtb[RS], pz[RS];
  T pk[RS], pq_[RS], pb = T(0.f), pv = T(0.f);
#pragma unroll
  for (int i = 0; i < RS; ++i) {
    const int kk = lane + 32 * i;
    dtb[i] = kk < dk ? dt_bias[head * dk + kk] : 0.f;
    pk[i] = pq_[i] = T(0.f);
    pz[i] = 0.f;
  }
  const int jj = blockIdx.x * DELTA_COLS + lane;   // the column whose value this lane stages
  auto fetch = [&](int t) {
    if (t >= len) return;
    const size_t m = (size_t)(row0 + t);
    const T* kr = k + m * stride + kvh * dk;
    const T* qr = q + m * stride + kvh * dk;
#pragma unroll
    for (int i = 0; i < RS; ++i) {
      const int kk = lane + 32 * i;
      if (kk < dk) {
        pk[i] = kr[kk];
        pq_[i] = qr[kk];
        pz[i] = z[m * z_stride + head * dk + kk];
      }
    }
    pb = b[m * b_stride + head];
    if (jj < dv) pv = v[m * stride + head * dv + jj];
  };
  fetch(warp);
  for (int t0 = 0; t0 < len; t0 += DELTA_L) {
    const int n = min(DELTA_L, len - t0);
    __syncthreads();   // the group before is consumed
    if (warp < n) {
      const int l = warp;
      float kv_[RS], qv_[RS], ssk = 0.f, ssq = 0.f;
#pragma unroll
      for (int i = 0; i < RS; ++i) {
        kv_[i] = mi_to_float(pk[i]);
        qv_[i] = mi_to_float(pq_[i]);
        ssk = fmaf(kv_[i], kv_[i], ssk);
        ssq = fmaf(qv_[i], qv_[i], ssq);
      }
      ssk = mi_warp_sum(ssk);
      ssq = mi_warp_sum(ssq);
      const float mk = 1.f / sqrtf(ssk + unit_eps), mq = q_scale / sqrtf(ssq + unit_eps);
      float kq = 0.f;
#pragma unroll
      for (int i = 0; i < RS; ++i) {
        const int kk = lane + 32 * i;
        float kn = 0.f, qn = 0.f, g = 1.f;
        if (kk < dk) {
          kn = kv_[i] * mk;
          qn = qv_[i] * mq;
          g = expf(-A * mi_softplus(pz[i] + dtb[i]));
        }
        ks[l * DKP + kk] = kn;
        qs[l * DKP + kk] = qn;
        gs[l * DKP + kk] = g;
        kq = fmaf(kn, qn, kq);
      }
      kq = mi_warp_sum(kq);
      if (lane == 0) {
        kqs[l] = kq;
        bs[l] = mi_sigmoid(mi_to_float(pb));
      }
      vs[l * DELTA_COLS + lane] = jj < dv ? mi_to_float(pv) : 0.f;
    }
    __syncthreads();
    fetch(t0 + DELTA_L + warp);
    for (int l = 0; l < n; ++l) {
      float kreg[R];
      float r0 = 0.f, r1 = 0.f, p0 = 0.f, p1 = 0.f;
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const int at = l * DKP + 4 * (part + DELTA_PARTS * i);
        const float4 g4 = *reinterpret_cast<const float4*>(gs + at);
        const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
        const float4 q4 = *reinterpret_cast<const float4*>(qs + at);
        float* si = s + 4 * i;
        float* ki = kreg + 4 * i;
        ki[0] = k4.x; ki[1] = k4.y; ki[2] = k4.z; ki[3] = k4.w;
        si[0] *= g4.x; si[1] *= g4.y; si[2] *= g4.z; si[3] *= g4.w;
        r0 = fmaf(si[0], k4.x, r0); r1 = fmaf(si[1], k4.y, r1);
        r0 = fmaf(si[2], k4.z, r0); r1 = fmaf(si[3], k4.w, r1);
        p0 = fmaf(si[0], q4.x, p0); p1 = fmaf(si[1], q4.y, p1);
        p0 = fmaf(si[2], q4.z, p0); p1 = fmaf(si[3], q4.w, p1);
      }
      float r = r0 + r1, pq = p0 + p1;
#pragma unroll
      for (int off = DELTA_NC; off < 32; off <<= 1) {
        r += __shfl_xor_sync(0xffffffffu, r, off);
        pq += __shfl_xor_sync(0xffffffffu, pq, off);
      }
      const float u = bs[l] * (vs[l * DELTA_COLS + warp * DELTA_NC + col] - r);
#pragma unroll
      for (int i = 0; i < R; ++i) s[i] = fmaf(kreg[i], u, s[i]);
      if (part == 0 && j < dv) o[(size_t)(row0 + t0 + l) * o_stride + head * dv + j] = fmaf(u, kqs[l], pq);
    }
  }
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = 4 * (part + DELTA_PARTS * i) + e;
      if (kk < dk && j < dv) S[(size_t)kk * dv + j] = s[4 * i + e];
    }
  // the convolution's next tail (the request's blocks share its channels): the last taps-1 of (old tail,
  // this portion's inputs); the convolution itself ran before this kernel and nothing else reads the tail here
  if (taps > 1) {
    const int n_blocks = gridDim.x * gridDim.y, block_id = blockIdx.y * gridDim.x + blockIdx.x;
    for (int c = block_id * 32 * DELTA_W + tid; c < C; c += n_blocks * 32 * DELTA_W) {
      float keep[MAX_TAPS];
#pragma unroll
      for (int j = 0; j < MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
          const int src = len - (taps - 1) + j;
          keep[j] = src >= 0 ? mi_to_float(xin[(size_t)(row0 + src) * xin_stride + c])
                             : st[(size_t)(taps - 1 + src) * C + c];
        }
      }
#pragma unroll
      for (int j = 0; j < MAX_TAPS - 1; ++j)
        if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
    }
  }
}

extern "C" int mi_delta_scan(const void* q, const void* k, const void* v, int stride, const float* z, int z_stride,
                             const float* dt_bias, const float* a_log, const void* b, int b_stride, float q_scale,
                             float unit_eps, float* state, long long state_stride, long long s_off,
                             const int* q_start, const int* q_len, const int* state_slot, float* o, int o_stride,
                             int n_requests, int heads, int kv_heads, int dk, int dv, const void* xin, int xin_stride,
                             int C, int taps, int dtype, cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (dk <= 0 || dk > 256 || dv <= 0) MI_REFUSE("delta: key size %d must lie in [1, 256], value size %d above 0", dk, dv);
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) MI_REFUSE("delta: %d heads cannot share %d key heads", heads, kv_heads);
  if (heads > 65535 || n_requests > 65535) MI_REFUSE("delta: too many heads or requests for one launch");
  if (taps < 1 || taps > MAX_TAPS) MI_REFUSE("delta: %d taps (1 to %d are taken)", taps, MAX_TAPS);
  dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, heads, n_requests), block(32, DELTA_W);
  const int dkp = dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256;   // DELTA_PARTS * R of the instance below
  const size_t smem = ((size_t)3 * DELTA_L * dkp + DELTA_L * DELTA_COLS + 2 * DELTA_L) * sizeof(float);
#define MI_GO(T, R)                                                                                                  \
  do {                                                                                                               \
    auto kern = delta_scan_kernel<T, R>;                                                                             \
    if (smem > 48 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    MI_LAUNCH(kern, grid, block, smem, stream, (const T*)q, (const T*)k, (const T*)v, stride, z, z_stride, dt_bias,  \
              a_log, (const T*)b, b_stride, q_scale, unit_eps, state, state_stride, s_off, q_start, q_len,          \
              state_slot, o, o_stride, heads, kv_heads, dk, dv, (const T*)xin, xin_stride, C, taps);                 \
  } while (0)
#define MI_GO_R(T)                  \
  do {                              \
    if (dk <= 32) MI_GO(T, 4);       \
    else if (dk <= 64) MI_GO(T, 8);  \
    else if (dk <= 128) MI_GO(T, 16);\
    else MI_GO(T, 32);               \
  } while (0)
  if (dtype == MI_DTYPE_F32) MI_GO_R(float);
  else if (dtype == MI_DTYPE_BF16) MI_GO_R(bf16);
  else MI_REFUSE("delta: unknown dtype %d", dtype);
#undef MI_GO_R
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------
// per-head RMS norm with a gain (shared by the heads: w_head = 0; one per head: w_head = dv), times an
// activated gate.  One warp per (token, head).  With tok_gates [M, heads, 3] a head of o has dv + 1
// columns, the last one a normaliser n, and the head is first divided by max(|n|, exp(-m)) + den_eps,
// m the third number of the token's and head's gates (a matrix memory with a running maximum).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void headnorm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ w,
                                     const T* __restrict__ g, int g_stride, T* __restrict__ out, int out_stride,
                                     int M, int heads, int dv, float eps, int act, float scale, int w_head,
                                     const float* __restrict__ tok_gates, float den_eps) {
  mi_pdl_enter();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)M * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit - (long long)t * heads);
  const float* src = o + (size_t)t * o_stride + (size_t)h * (dv + (tok_gates ? 1 : 0));
  float inv_den = 1.f;
  if (tok_gates) inv_den = 1.f / (fmaxf(fabsf(src[dv]), expf(-tok_gates[((size_t)t * heads + h) * 3 + 2])) + den_eps);
  w += (size_t)h * w_head;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float v = src[c] * inv_den;
    ss += v * v;
  }
  ss = mi_warp_sum(ss);
  const float mult = inv_den / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    float a = 1.f;
    if (act) {
      const float gv = mi_to_float(g[(size_t)t * g_stride + h * dv + c]);
      const float sg = 1.f / (1.f + expf(-gv));
      a = act == 2 ? gv * sg : sg;
    }
    out[(size_t)t * out_stride + h * dv + c] = mi_from_float<T>(src[c] * mult * w[c] * a * scale);
  }
}

extern "C" int mi_headnorm_gate(const float* o, int o_stride, const float* w, const void* g, int g_stride,
                                void* out, int out_stride, int M, int heads, int dv, float eps, int act,
                                float scale, int w_head, const float* tok_gates, float den_eps, int dtype,
                                cudaStream_t stream) {
  if (M <= 0 || heads <= 0) return 0;
  if (act < 0 || act > 2) MI_REFUSE("headnorm_gate: unknown activation %d", act);
  const long long units = (long long)M * heads;
  const long long blocks = (units + 3) / 4;
  if (blocks > 0x7fffffffLL) MI_REFUSE("headnorm_gate: too many blocks for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((headnorm_gate_kernel<float>), (unsigned)blocks, 128, 0, stream, o, o_stride, w, (const float*)g,
              g_stride, (float*)out, out_stride, M, heads, dv, eps, act, scale, w_head, tok_gates, den_eps);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((headnorm_gate_kernel<bf16>), (unsigned)blocks, 128, 0, stream, o, o_stride, w, (const bf16*)g,
              g_stride, (bf16*)out, out_stride, M, heads, dv, eps, act, scale, w_head, tok_gates, den_eps);
  else
    MI_REFUSE("headnorm_gate: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}
