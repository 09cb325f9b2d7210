// Kernels around an fp32 residual stream that takes several addends at once.
//
//   mi_embedding_pair_hash   stream[t, :] = float(table[id_t, :]) + float(pair_table[row_t, :])     (fp32 out)
//                            row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets, and row `buckets`
//                            (the table's last row) for a sequence's first token (position 0).  prev_t is
//                            the token before t: the one before it in the step's portion, or, for a
//                            portion's first token, the request's entry of last_token[] (per request
//                            slot), which the block of that first token then replaces by the portion's
//                            last token.
//   mi_embedding_rmsnorm     stream[t, :] = x * rsqrt(mean(x^2) + eps) * gain with x = float(table[id_t, :]): an
//                            embedding that is normalised before it becomes the fp32 stream.
//   mi_add_rmsnorm_multi     r = stream_in[src] + (float(add1[src]) + float(add2[src])) + add32[src] + row_add
//                            (fp32; every addend optional); stream_out[i] = r (if given; may be stream_in
//                            when there is no gather); out[i] = T(r * rsqrt(mean(r^2) + eps) * gain).
//                            One block per output row; src = rows[i] when a gather list is given, else i.
//   mi_glu_mul_pairs         out[m, i] = T(act(gu[m, 2i]) * gu[m, 2i + 1]), act = SiLU (1) or the tanh form
//                            of GELU (2): the layout of a merged gate/up product whose rows alternate.
//   mi_scaled_norm_add       a branch whose norm stands behind it: stream[t, :] += mult * y * rsqrt(mean(y^2) + eps)
//                            * gain with y = float(branch[t, :]), in place (fp32), and copy[t, :] = T(stream[t, :]),
//                            what the next branch's products read.  Without a branch: the copy alone.
//   mi_token_gate            out[t, c] = T(gelu_tanh(z[t, c]) * float(table[id_t, col0 + c])): a gate times the
//                            columns [col0, col0 + n) of a token's row of a table.
//   mi_scale_f32             x *= s in place (fp32).
#include "common.cuh"

MI_DEFINE_ERROR_API()

template <typename T>
__global__ void embedding_pair_hash_kernel(const T* __restrict__ table, const T* __restrict__ pair_table,
                                           const int* __restrict__ ids, const int* __restrict__ positions,
                                           const int* __restrict__ q_start, const int* __restrict__ q_len,
                                           const int* __restrict__ state_slot, int* __restrict__ last_token,
                                           int n_requests, float* __restrict__ out, int H, int V, int buckets,
                                           long long mul_prev, long long mul_cur) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  int lo = 0, hi = n_requests - 1;      // the request of token t: the last one whose portion starts at or before t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (q_start[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int first = q_start[lo];
  const int id = ids[t];
  const int slot = state_slot[lo];
  const int prev = t > first ? ids[t - 1] : last_token[slot];
  __syncthreads();                      // every thread has read the entry before one of them replaces it
  if (t == first && threadIdx.x == 0) last_token[slot] = ids[first + q_len[lo] - 1];
  float* dst = out + (size_t)t * H;
  if ((unsigned)id >= (unsigned)V) {    // the step function validates ids; this keeps a fault visible
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
    return;
  }
  long long row = buckets;
  if (positions[t] != 0) {
    row = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
    if (row < 0) row += buckets;
  }
  const T* a = table + (size_t)id * H;
  const T* b = pair_table + (size_t)row * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = mi_to_float(a[i]) + mi_to_float(b[i]);
}

extern "C" int mi_embedding_pair_hash(const void* table, const void* pair_table, const int* ids, const int* positions,
                                      const int* q_start, const int* q_len, const int* state_slot, int* last_token,
                                      int n_requests, float* out, int M, int H, int V, int buckets,
                                      long long mul_prev, long long mul_cur, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || V <= 0 || buckets <= 0 || n_requests <= 0) MI_REFUSE("embedding: bad sizes H=%d V=%d buckets=%d", H, V, buckets);
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((embedding_pair_hash_kernel<float>), M, threads, 0, stream, (const float*)table, (const float*)pair_table,
              ids, positions, q_start, q_len, state_slot, last_token, n_requests, out, H, V, buckets, mul_prev, mul_cur);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((embedding_pair_hash_kernel<bf16>), M, threads, 0, stream, (const bf16*)table, (const bf16*)pair_table,
              ids, positions, q_start, q_len, state_slot, last_token, n_requests, out, H, V, buckets, mul_prev, mul_cur);
  else
    MI_REFUSE("embedding: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

template <typename T>
__global__ void add_rmsnorm_multi_kernel(const float* __restrict__ stream_in, const T* __restrict__ add1,
                                         const T* __restrict__ add2, const float* __restrict__ add32,
                                         const float* __restrict__ row_add, float* __restrict__ stream_out,
                                         const int* __restrict__ rows, const float* __restrict__ gain,
                                         T* __restrict__ out, int H, float eps) {
  mi_pdl_enter();
  extern __shared__ float smem[];
  float* red = smem;        // 32 floats
  float* row = smem + 32;   // H floats
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  const float* sr = stream_in ? stream_in + (size_t)src * H : nullptr;
  const T* a1 = add1 ? add1 + (size_t)src * H : nullptr;
  const T* a2 = add2 ? add2 + (size_t)src * H : nullptr;
  const float* a3 = add32 ? add32 + (size_t)src * H : nullptr;
  float sq = 0.f;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    float branches = 0.f;
    if (a1) branches = mi_to_float(a1[k]);
    if (a2) branches += mi_to_float(a2[k]);
    float r = sr ? sr[k] + branches : branches;
    if (a3) r += a3[k];
    if (row_add) r += row_add[k];
    row[k] = r;
    sq += r * r;
  }
  const float rstd = 1.f / sqrtf(mi_block_sum(sq, red) / (float)H + eps);
  float* so = stream_out ? stream_out + (size_t)i * H : nullptr;
  T* o = out + (size_t)i * H;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    const float r = row[k];
    if (so) so[k] = r;
    o[k] = mi_from_float<T>(r * rstd * gain[k]);
  }
}

extern "C" int mi_add_rmsnorm_multi(const float* stream_in, const void* add1, const void* add2, const float* add32,
                                    const float* row_add, float* stream_out, const int* rows, const float* gain,
                                    void* out, int M, int H, float eps, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0) MI_REFUSE("rmsnorm: bad width %d", H);
  if (rows && stream_out) MI_REFUSE("rmsnorm: a gathered norm does not write the stream");
  const size_t smem = (32 + (size_t)H) * sizeof(float);
  if (smem > 200 * 1024) MI_REFUSE("rmsnorm: a row of %d floats does not fit in shared memory", H);
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define MI_GO(T)                                                                                          \
  do {                                                                                                    \
    auto kern = add_rmsnorm_multi_kernel<T>;                                                              \
    if (smem > 48 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                \
    }                                                                                                     \
    MI_LAUNCH(kern, M, threads, smem, stream, stream_in, (const T*)add1, (const T*)add2, add32, row_add,   \
              stream_out, rows, gain, (T*)out, H, eps);                                                   \
  } while (0)
  if (dtype == MI_DTYPE_F32) MI_GO(float);
  else if (dtype == MI_DTYPE_BF16) MI_GO(bf16);
  else MI_REFUSE("rmsnorm: unknown dtype %d", dtype);
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}

__device__ __forceinline__ float glu_act(float g, int act) {
  if (act == 2) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(inner));
  }
  return g / (1.f + expf(-g));
}

template <typename T>
__global__ void glu_mul_pairs_kernel(const T* __restrict__ gu, T* __restrict__ out, int M, int I, int act) {
  mi_pdl_enter();
  const size_t n = (size_t)M * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
    out[idx] = mi_from_float<T>(glu_act(mi_to_float(gu[2 * idx]), act) * mi_to_float(gu[2 * idx + 1]));
}

// bfloat16, eight outputs per thread: two 16-byte loads, one 16-byte store
__global__ void glu_mul_pairs8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, size_t n8, int act) {
  mi_pdl_enter();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n8; idx += (size_t)gridDim.x * blockDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(gu) + 2 * idx;
    const uint4 a = in[0], b = in[1];
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};   // each word: (gate, up) of one output
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j]));
      const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j + 1]));
      const __nv_bfloat162 o = __floats2bfloat162_rn(glu_act(p0.x, act) * p0.y, glu_act(p1.x, act) * p1.y);
      r[j] = *reinterpret_cast<const uint32_t*>(&o);
    }
    reinterpret_cast<uint4*>(out)[idx] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

extern "C" int mi_glu_mul_pairs(const void* gu, void* out, int M, int I, int act, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (I <= 0) MI_REFUSE("glu_mul: bad width %d", I);
  if (act != 1 && act != 2) MI_REFUSE("glu_mul: unknown activation %d", act);
  const size_t n = (size_t)M * I;
  if (dtype == MI_DTYPE_BF16 && I % 8 == 0 && mi_aligned(gu, 16) && mi_aligned(out, 16)) {
    const size_t n8 = n / 8;
    const int blocks = (int)((n8 + 255) / 256 < 8192 ? (n8 + 255) / 256 : 8192);
    MI_LAUNCH((glu_mul_pairs8_kernel), blocks, 256, 0, stream, (const bf16*)gu, (bf16*)out, n8, act);
    MI_RETURN_LAUNCH_STATUS();
  }
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((glu_mul_pairs_kernel<float>), blocks, 256, 0, stream, (const float*)gu, (float*)out, M, I, act);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((glu_mul_pairs_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gu, (bf16*)out, M, I, act);
  else
    MI_REFUSE("glu_mul: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}


template <typename T>
__global__ void embedding_rmsnorm_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                         const float* __restrict__ gain, float* __restrict__ out, int H, int V,
                                         float eps) {
  mi_pdl_enter();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * H;
  if ((unsigned)id >= (unsigned)V) {    // the step function validates ids; this keeps a fault visible
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)id * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = mi_to_float(src[i]);
    ss += v * v;
  }
  const float mult = 1.f / sqrtf(mi_block_sum(ss, red) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = mi_to_float(src[i]) * mult * gain[i];
}

extern "C" int mi_embedding_rmsnorm(const void* table, const int* ids, const float* gain, float* out, int M, int H,
                                    int V, float eps, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || V <= 0) MI_REFUSE("embedding: bad sizes H=%d V=%d", H, V);
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((embedding_rmsnorm_kernel<float>), M, threads, 0, stream, (const float*)table, ids, gain, out, H, V, eps);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((embedding_rmsnorm_kernel<bf16>), M, threads, 0, stream, (const bf16*)table, ids, gain, out, H, V, eps);
  else
    MI_REFUSE("embedding: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}


template <typename T>
__global__ void scaled_norm_add_kernel(float* __restrict__ stream, const T* __restrict__ branch, int branch_stride,
                                       const float* __restrict__ gain, float eps, float mult, T* __restrict__ copy,
                                       int H) {
  mi_pdl_enter();
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* sr = stream + (size_t)t * H;
  T* cp = copy ? copy + (size_t)t * H : nullptr;
  if (!branch) {
    for (int k = threadIdx.x; k < H; k += blockDim.x) cp[k] = mi_from_float<T>(sr[k]);
    return;
  }
  const T* y = branch + (size_t)t * branch_stride;
  float sq = 0.f;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    const float v = mi_to_float(y[k]);
    sq += v * v;
  }
  const float rstd = 1.f / sqrtf(mi_block_sum(sq, red) / (float)H + eps);
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    const float r = sr[k] + mult * (mi_to_float(y[k]) * rstd * gain[k]);
    sr[k] = r;
    if (cp) cp[k] = mi_from_float<T>(r);
  }
}

// the same with four elements per access (rows of whole 16-byte pieces); the sums run in the same order
// for a row whatever else the launch holds
template <typename T>
__global__ void scaled_norm_add4_kernel(float* __restrict__ stream, const T* __restrict__ branch, int branch_stride,
                                        const float* __restrict__ gain, float eps, float mult, T* __restrict__ copy,
                                        int H) {
  mi_pdl_enter();
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* sr = stream + (size_t)t * H;
  T* cp = copy ? copy + (size_t)t * H : nullptr;
  float f[4], r[4], g[4];
  if (!branch) {
    for (int k = 4 * threadIdx.x; k < H; k += 4 * blockDim.x) {
      Vec4<float> a;
      a.load(sr + k);
      a.get(r);
      Vec4<T> o;
      o.set(r);
      o.store(cp + k);
    }
    return;
  }
  const T* y = branch + (size_t)t * branch_stride;
  float sq = 0.f;
  for (int k = 4 * threadIdx.x; k < H; k += 4 * blockDim.x) {
    Vec4<T> a;
    a.load(y + k);
    a.get(f);
    sq += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
  }
  const float rstd = 1.f / sqrtf(mi_block_sum(sq, red) / (float)H + eps);
  for (int k = 4 * threadIdx.x; k < H; k += 4 * blockDim.x) {
    Vec4<T> a;
    a.load(y + k);
    a.get(f);
    Vec4<float> b, w;
    b.load(sr + k);
    b.get(r);
    w.load(gain + k);
    w.get(g);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = r[i] + mult * (f[i] * rstd * g[i]);
    b.set(r);
    b.store(sr + k);
    if (cp) {
      Vec4<T> o;
      o.set(r);
      o.store(cp + k);
    }
  }
}

extern "C" int mi_scaled_norm_add(float* stream, const void* branch, int branch_stride, const float* gain, float eps,
                                  float mult, void* copy, int M, int H, int dtype, cudaStream_t stream_) {
  if (M <= 0) return 0;
  if (H <= 0) MI_REFUSE("norm_add: bad width %d", H);
  if (!stream || (branch && !gain) || (!branch && !copy)) MI_REFUSE("norm_add: a stream and a branch with its gain, or a copy to make");
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (H % 4 == 0 && branch_stride % 4 == 0 && mi_aligned(stream, 16) && mi_aligned(branch, 16) && mi_aligned(gain, 16) &&
      mi_aligned(copy, 16)) {
    const int t4 = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (dtype == MI_DTYPE_F32)
      MI_LAUNCH((scaled_norm_add4_kernel<float>), M, t4, 0, stream_, stream, (const float*)branch, branch_stride, gain,
                eps, mult, (float*)copy, H);
    else if (dtype == MI_DTYPE_BF16)
      MI_LAUNCH((scaled_norm_add4_kernel<bf16>), M, t4, 0, stream_, stream, (const bf16*)branch, branch_stride, gain,
                eps, mult, (bf16*)copy, H);
    else
      MI_REFUSE("norm_add: unknown dtype %d", dtype);
    MI_RETURN_LAUNCH_STATUS();
  }
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((scaled_norm_add_kernel<float>), M, threads, 0, stream_, stream, (const float*)branch, branch_stride, gain,
              eps, mult, (float*)copy, H);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((scaled_norm_add_kernel<bf16>), M, threads, 0, stream_, stream, (const bf16*)branch, branch_stride, gain,
              eps, mult, (bf16*)copy, H);
  else
    MI_REFUSE("norm_add: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

template <typename TZ, typename T>
__global__ void token_gate_kernel(const TZ* __restrict__ z, int z_stride, const T* __restrict__ table, int table_stride,
                                  const int* __restrict__ ids, int V, int col0, T* __restrict__ out, int M, int n) {
  mi_pdl_enter();
  const size_t total = (size_t)M * n;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / n), c = (int)(idx - (size_t)t * n);
    const int id = ids[t];
    float e = __int_as_float(0x7fc00000);      // the step function validates ids; this keeps a fault visible
    if ((unsigned)id < (unsigned)V) e = mi_to_float(table[(size_t)id * table_stride + col0 + c]);
    out[idx] = mi_from_float<T>(glu_act(mi_to_float(z[(size_t)t * z_stride + c]), 2) * e);
  }
}

// z_dtype: the gate's pre-activations are fp32 or in the compute dtype
extern "C" int mi_token_gate(const void* z, int z_stride, int z_dtype, const void* table, int table_stride,
                             const int* ids, int V, int col0, void* out, int M, int n, int dtype, cudaStream_t stream) {
  if (M <= 0 || n <= 0) return 0;
  if (col0 < 0 || col0 + n > table_stride || V <= 0) MI_REFUSE("token_gate: columns %d..%d of a row of %d", col0, col0 + n, table_stride);
  const size_t total = (size_t)M * n;
  const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  if (dtype == MI_DTYPE_F32 && z_dtype == MI_DTYPE_F32)
    MI_LAUNCH((token_gate_kernel<float, float>), blocks, 256, 0, stream, (const float*)z, z_stride, (const float*)table,
              table_stride, ids, V, col0, (float*)out, M, n);
  else if (dtype == MI_DTYPE_BF16 && z_dtype == MI_DTYPE_F32)
    MI_LAUNCH((token_gate_kernel<float, bf16>), blocks, 256, 0, stream, (const float*)z, z_stride, (const bf16*)table,
              table_stride, ids, V, col0, (bf16*)out, M, n);
  else if (dtype == MI_DTYPE_BF16 && z_dtype == MI_DTYPE_BF16)
    MI_LAUNCH((token_gate_kernel<bf16, bf16>), blocks, 256, 0, stream, (const bf16*)z, z_stride, (const bf16*)table,
              table_stride, ids, V, col0, (bf16*)out, M, n);
  else
    MI_REFUSE("token_gate: unsupported dtypes %d (table) and %d (gate)", dtype, z_dtype);
  MI_RETURN_LAUNCH_STATUS();
}

__global__ void scale_f32_kernel(float* __restrict__ x, size_t n, float s) {
  mi_pdl_enter();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
    x[idx] *= s;
}

extern "C" int mi_scale_f32(float* x, long long n, float s, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  MI_LAUNCH((scale_f32_kernel), blocks, 256, 0, stream, x, (size_t)n, s);
  MI_RETURN_LAUNCH_STATUS();
}
