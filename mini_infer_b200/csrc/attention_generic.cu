// Attention over the paged key/value cache, any portion length, CUDA cores, fp32 math.
//
// This is the kernel of the 32-bit path and the plain twin of the tensor-core
// kernels.  One block takes 16 consecutive query tokens of one request and one query
// head, walks that request's keys in chunks of 32 (always cut at absolute multiples of
// 32, so a row's arithmetic never depends on what else is in the batch), and keeps an
// online softmax in fp32.  Keys and values are fetched through the block table; a
// query at absolute position p sees keys j with  max(0, p - window + 1) <= j <= p
// (window = 0: all keys up to p), and with chunk > 0 only those of its own chunk of positions,
// j >= (p / chunk) * chunk.  Keys and values may have different sizes per head (d for
// queries and keys, dv for values and the output); keys of any size that fits in shared memory
// and values up to 512 are taken, sizes that are no multiple of 4 element by element.
//
// Three optional extras.  `sinks` [nq]: the softmax's denominator also holds exp(sinks[h]), a
// score without a key or a value that is not scaled and counts once.  `slopes` [nq]: the scaled
// score of query i and key j is lowered by slopes[h] * (i - j).  `v_prefix`: there is no value
// cache; the value of a key is the first dv numbers of the key's own row (dv <= d).
//
// Layouts
//   q    [tokens, q_stride]   head h at columns [h*d, (h+1)*d)
//   out  [tokens, out_stride] head h at columns [h*dv, (h+1)*dv)
//   kcache [pages, nkv, page_size, d], vcache [pages, nkv, page_size, dv]: the page_size keys of
//                  a page lie together per key/value head; the 16-byte chunks of a row are permuted
//                  by the key's in-page offset (mi_swizzled in common.cuh; rows that are no whole
//                  number of chunks are not permuted, mi_swizzle_mask_rows)
//   block_table [rows, bt_stride] page ids; request b uses row table_rows[b] (row b when
//                  table_rows is null);  q_start / q_len / kv_len [requests]
//   tile_req / tile_tok0 [tiles]: request and first token (within the portion) of a tile
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define BQ 16
#define BK 32
#define NTHREADS 128

template <typename T, int DMAX>
__global__ void __launch_bounds__(NTHREADS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ kcache, const T* __restrict__ vcache,
                         const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ table_rows, int page_size,
                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                         const int* __restrict__ kv_len, const int* __restrict__ tile_req,
                         const int* __restrict__ tile_tok0, int nq, int nkv, int d, int dv, float scale,
                         int window, int chunk, const float* __restrict__ sinks, const float* __restrict__ slopes,
                         int v_prefix) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ __align__(16) float smem[];
  float* Vs = smem;                       // [BK][dvp], dvp = dv rounded up to 4 (nothing with v_prefix)
  const int dvp = (dv + 3) & ~3;
  float* Qs = Vs + (v_prefix ? 0 : BK * dvp);   // [BQ][d]
  float* Ks = Qs + BQ * d;                // [BK][d + 1]
  float* Ss = Ks + BK * (d + 1);          // [BQ][BK]
  int* rowbase = reinterpret_cast<int*>(Ss + BQ * BK);  // [BK] element offset / d of each key row, -1: none
  int* rowswz = rowbase + BK;                            // [BK] chunk permutation of each key row
  constexpr int EPC = 16 / (int)sizeof(T);
  const int swz_mask = mi_swizzle_mask_rows(d, (int)sizeof(T));
  const int swz_mask_v = mi_swizzle_mask_rows(dv, (int)sizeof(T));

  const int tid = threadIdx.x;
  const int tile = blockIdx.x / nq, h = blockIdx.x - tile * nq;   // all heads of a tile, then the next tile (the caller lists long tiles first)
  const int kvh = h / (nq / nkv);
  const int b = tile_req[tile], tok0 = tile_tok0[tile];
  const int ql = q_len[b], kl = kv_len[b], qs = q_start[b];
  const int trow = table_rows ? table_rows[b] : b;   // the request's row of the block table
  const int rows = min(BQ, ql - tok0);
  const int p0 = kl - ql + tok0;  // absolute position of the tile's first query
  const int j_end = p0 + rows;    // one past the last visible key
  int j_lo = window > 0 ? max(0, p0 - window + 1) : 0;   // the first row's bound is the lowest of the tile
  if (chunk > 0) j_lo = max(j_lo, (p0 / chunk) * chunk);
  const int dp = d + 1;
  const float* Vrows = v_prefix ? Ks : Vs;   // where the PV product finds a key's value, and its row pitch
  const int vpitch = v_prefix ? dp : dvp;
  const float slope = slopes ? slopes[h] : 0.f;

  for (int idx = tid; idx < BQ * d; idx += NTHREADS) {
    const int r = idx / d, k = idx - r * d;
    Qs[idx] = r < rows ? mi_to_float(q[(size_t)(qs + tok0 + r) * q_stride + h * d + k]) : 0.f;
  }

  const int r = tid >> 3, c = tid & 7;
  const int prow = p0 + r;
  int lo_r = window > 0 ? max(0, prow - window + 1) : 0;
  if (chunk > 0) lo_r = max(lo_r, (prow / chunk) * chunk);
  float m_i = -INFINITY, l_i = 0.f;
  float acc[DMAX / 8];
#pragma unroll
  for (int e = 0; e < DMAX / 8; ++e) acc[e] = 0.f;
  const int ne = (dv + 7) >> 3;

  for (int j0 = (j_lo / BK) * BK; j0 < j_end; j0 += BK) {
    __syncthreads();  // previous chunk fully consumed (and Qs written, first time)
    if (tid < BK) {
      const int j = j0 + tid;
      int base = -1;
      if (j >= j_lo && j < j_end) {
        const int page = block_table[(size_t)trow * bt_stride + j / page_size];
        base = (page * nkv + kvh) * page_size + j % page_size;
      }
      rowbase[tid] = base;
      rowswz[tid] = (j % page_size);
    }
    __syncthreads();
    if ((d & 3) == 0) {
      const int d4 = d >> 2;
      for (int idx = tid; idx < BK * d4; idx += NTHREADS) {
        const int jj = idx / d4, k4 = (idx - jj * d4) << 2;
        const int base = rowbase[jj];
        float kf[4] = {0.f, 0.f, 0.f, 0.f};
        if (base >= 0) {
          const size_t off = (size_t)base * d + ((((k4 / EPC) ^ (rowswz[jj] & swz_mask)) * EPC) + (k4 % EPC));
          Vec4<T> kv;
          kv.load(kcache + off);
          kv.get(kf);
        }
        float* kd = Ks + jj * dp + k4;
        kd[0] = kf[0]; kd[1] = kf[1]; kd[2] = kf[2]; kd[3] = kf[3];
      }
    } else {
      for (int idx = tid; idx < BK * d; idx += NTHREADS) {
        const int jj = idx / d, k = idx - jj * d;
        const int base = rowbase[jj];
        Ks[jj * dp + k] = base >= 0 ? mi_to_float(kcache[(size_t)base * d + mi_swizzled(k, rowswz[jj], swz_mask, EPC)]) : 0.f;
      }
    }
    if (v_prefix) {
      // the values are the keys' own first columns, already in Ks
    } else if ((dv & 3) == 0) {
      const int d4 = dv >> 2;
      for (int idx = tid; idx < BK * d4; idx += NTHREADS) {
        const int jj = idx / d4, k4 = (idx - jj * d4) << 2;
        const int base = rowbase[jj];
        float vf[4] = {0.f, 0.f, 0.f, 0.f};
        if (base >= 0) {
          const size_t off = (size_t)base * dv + ((((k4 / EPC) ^ (rowswz[jj] & swz_mask_v)) * EPC) + (k4 % EPC));
          Vec4<T> vv;
          vv.load(vcache + off);
          vv.get(vf);
        }
        *reinterpret_cast<float4*>(Vs + jj * dvp + k4) = make_float4(vf[0], vf[1], vf[2], vf[3]);
      }
    } else {
      for (int idx = tid; idx < BK * dv; idx += NTHREADS) {
        const int jj = idx / dv, k = idx - jj * dv;
        const int base = rowbase[jj];
        Vs[jj * dvp + k] = base >= 0 ? mi_to_float(vcache[(size_t)base * dv + mi_swizzled(k, rowswz[jj], swz_mask_v, EPC)]) : 0.f;
      }
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* qrow = Qs + r * d;
    for (int k = 0; k < d; ++k) {
      const float qv = qrow[k];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) s[jj] = fmaf(qv, Ks[(c + 8 * jj) * dp + k], s[jj]);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = j0 + c + 8 * jj;
      const bool ok = (r < rows) && (j <= prow) && (j >= lo_r);
      s[jj] = ok ? s[jj] * scale - slope * (float)(prow - j) : -INFINITY;
      mx = fmaxf(mx, s[jj]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    const float m_new = fmaxf(m_i, mx);
    float alpha = 1.f, psum = 0.f;
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    if (m_new != -INFINITY) {
      alpha = expf(m_i - m_new);  // m_i = -inf gives 0
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        p[jj] = expf(s[jj] - m_new);  // masked entries give 0
        psum += p[jj];
      }
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    psum += __shfl_xor_sync(0xffffffffu, psum, 4);
    l_i = l_i * alpha + psum;
    m_i = m_new;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) Ss[r * BK + c + 8 * jj] = p[jj];
#pragma unroll
    for (int e = 0; e < DMAX / 8; ++e) acc[e] *= alpha;
    __syncthreads();
    for (int j = 0; j < BK; ++j) {
      const float pj = Ss[r * BK + j];
      const float* vrow = Vrows + j * vpitch + c;
#pragma unroll
      for (int e = 0; e < DMAX / 8; ++e)
        if (e < ne && c + 8 * e < dv) acc[e] = fmaf(pj, vrow[8 * e], acc[e]);
    }
  }
  if (sinks && r < rows) {
    // the sink joins the denominator once, on the scale of the larger of itself and the row's maximum
    const float sink = sinks[h];
    const float m_f = fmaxf(m_i, sink);
    const float keep = (m_i == -INFINITY) ? 0.f : expf(m_i - m_f);
    l_i = l_i * keep + expf(sink - m_f);
#pragma unroll
    for (int e = 0; e < DMAX / 8; ++e) acc[e] *= keep;
  }
  if (r < rows && l_i > 0.f) {
    const float inv = 1.f / l_i;
    T* orow = out + (size_t)(qs + tok0 + r) * out_stride + h * dv + c;
#pragma unroll
    for (int e = 0; e < DMAX / 8; ++e)
      if (e < ne && c + 8 * e < dv) orow[8 * e] = mi_from_float<T>(acc[e] * inv);
  }
}

template <typename T, int DMAX>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                  const void* vcache, const int* block_table, int bt_stride, const int* table_rows, int page_size,
                  const int* q_start, const int* q_len, const int* kv_len, const int* tile_req,
                  const int* tile_tok0, int n_tiles, int nq, int nkv, int d, int dv, float scale, int window,
                  int chunk, const float* sinks, const float* slopes, int v_prefix, cudaStream_t stream) {
  const size_t smem = ((v_prefix ? 0 : (size_t)BK * ((dv + 3) & ~3)) + (size_t)BQ * d + (size_t)BK * (d + 1) + BQ * BK) *
                          sizeof(float) + 2 * BK * sizeof(int);
  auto kern = attention_generic_kernel<T, DMAX>;
  if (smem > 227 * 1024) return MI_REFUSED - 1;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((unsigned)(n_tiles * nq));
  MI_LAUNCH((kern), grid, NTHREADS, smem, stream, (const T*)q, q_stride, (T*)out, out_stride, (const T*)kcache,
                                         (const T*)vcache, block_table, bt_stride, table_rows, page_size, q_start,
                                         q_len, kv_len, tile_req, tile_tok0, nq, nkv, d, dv, scale, window, chunk, sinks,
                                         slopes, v_prefix);
  return 0;
}

extern "C" int mi_attention_generic_tile_tokens() { return BQ; }

extern "C" int mi_attention_generic_masked(const void* q, int q_stride, void* out, int out_stride,
                                           const void* kcache, const void* vcache, const int* block_table,
                                           int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                           const int* q_len, const int* kv_len, const int* tile_req,
                                           const int* tile_tok0, int n_tiles, int nq, int nkv, int d, int dv,
                                           float scale, int window, int chunk, const float* sinks,
                                           const float* slopes, int v_prefix, int dtype, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (chunk < 0) MI_REFUSE("attention: bad chunk size %d", chunk);
  if (d <= 0 || d > 1024 || dv <= 0 || dv > 512)
    MI_REFUSE("attention: head sizes %d (keys, up to 1024) and %d (values, up to 512) are not taken", d, dv);
  if (v_prefix && dv > d) MI_REFUSE("attention: values of %d cannot be the first columns of keys of %d", dv, d);
  if (!v_prefix && !vcache) MI_REFUSE("attention: no value cache");
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0)
    MI_REFUSE("attention: %d query heads cannot share %d key/value heads", nq, nkv);
  if ((long long)n_tiles * nq > 0x7fffffffLL) MI_REFUSE("attention: too many blocks for one launch");
  if (page_size <= 0 || window < 0) MI_REFUSE("attention: bad page size %d or window %d", page_size, window);
  if (!mi_aligned(kcache, 16) || !mi_aligned(vcache, 16)) MI_REFUSE("attention: cache must be 16-byte aligned");
  int rc;
#define MI_GO(T, DMAX)                                                                              \
  rc = launch<T, DMAX>(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride,        \
                       table_rows, page_size, q_start, q_len, kv_len, tile_req, tile_tok0, n_tiles, nq, nkv, d, dv, \
                       scale, window, chunk, sinks, slopes, v_prefix, stream)
  if (dtype == MI_DTYPE_F32) {
    if (dv <= 64) MI_GO(float, 64);
    else if (dv <= 128) MI_GO(float, 128);
    else if (dv <= 256) MI_GO(float, 256);
    else MI_GO(float, 512);
  } else if (dtype == MI_DTYPE_BF16) {
    if (dv <= 64) MI_GO(bf16, 64);
    else if (dv <= 128) MI_GO(bf16, 128);
    else if (dv <= 256) MI_GO(bf16, 256);
    else MI_GO(bf16, 512);
  } else {
    MI_REFUSE("attention: unknown dtype %d", dtype);
  }
#undef MI_GO
  if (rc == MI_REFUSED - 1) MI_REFUSE("attention: keys of %d and values of %d do not fit in shared memory", d, dv);
  if (rc) return rc;
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_attention_generic_ext(const void* q, int q_stride, void* out, int out_stride,
                                        const void* kcache, const void* vcache, const int* block_table,
                                        int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                        const int* q_len, const int* kv_len, const int* tile_req,
                                        const int* tile_tok0, int n_tiles, int nq, int nkv, int d, int dv,
                                        float scale, int window, const float* sinks, const float* slopes,
                                        int v_prefix, int dtype, cudaStream_t stream) {
  return mi_attention_generic_masked(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride, table_rows,
                                     page_size, q_start, q_len, kv_len, tile_req, tile_tok0, n_tiles, nq, nkv, d, dv,
                                     scale, window, 0, sinks, slopes, v_prefix, dtype, stream);
}

extern "C" int mi_attention_generic_kv(const void* q, int q_stride, void* out, int out_stride,
                                       const void* kcache, const void* vcache, const int* block_table,
                                       int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                       const int* q_len, const int* kv_len, const int* tile_req,
                                       const int* tile_tok0, int n_tiles, int nq, int nkv, int d, int dv,
                                       float scale, int window, int dtype, cudaStream_t stream) {
  return mi_attention_generic_ext(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride, table_rows,
                                  page_size, q_start, q_len, kv_len, tile_req, tile_tok0, n_tiles, nq, nkv, d, dv,
                                  scale, window, nullptr, nullptr, 0, dtype, stream);
}

// keys and values of one size, a multiple of 16 (what the tensor-core kernels take as well)
extern "C" int mi_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                    const void* kcache, const void* vcache, const int* block_table,
                                    int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                    const int* q_len, const int* kv_len, const int* tile_req,
                                    const int* tile_tok0, int n_tiles, int nq, int nkv, int d,
                                    float scale, int window, int dtype, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (d <= 0 || d % 16 != 0 || d > 256)
    MI_REFUSE("attention: head size %d is not a multiple of 16 in [16, 256]", d);
  return mi_attention_generic_kv(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride, table_rows,
                                 page_size, q_start, q_len, kv_len, tile_req, tile_tok0, n_tiles, nq, nkv, d, d,
                                 scale, window, dtype, stream);
}
