// What stands between an attention's input projection and the attention itself, for two kinds
// of attention.  Both kernels take the tokens one by one (a block, or a few blocks that share the
// heads, per token) and read column ranges of one packed
// projection [tokens, stride]; norms, angles, sines and cosines are fp32 or better, every value
// is rounded once.
//
//   mi_qk_bias_norm_store   queries and keys get a bias per column (optional) and then an RMS norm over
//                           the head with one gain shared by the heads (optional: x / sqrt(mean(x^2) + eps)
//                           * gain); q and k are written back in place, k goes to its cache page.  The
//                           values are either the keys as projected (with their bias, before the norm:
//                           values_are_keys) or a column range of their own; they go to the value pages.
//   mi_latent_prepare       for an attention whose keys and values are expanded from a low-rank latent and
//                           that is computed in the latent's space: the latent c (`rank` columns) gets an
//                           RMS norm with a gain; one key part shared by all heads (`rot_dim` columns behind
//                           c) is rotated by the token's position; the cache row of the token is
//                           [c normed, key part rotated].  Every query head's own rotated part (`rot_dim`
//                           columns at q_rot_off within the head) is rotated too and written behind the
//                           `rank` columns of that head in `qfull` [tokens, heads, rank + rot_dim], whose
//                           first `rank` columns per head the caller fills with the query mapped into the
//                           latent's space.
//                           Rotation, half layout: among the first `rot` of the rot_dim dimensions, i pairs
//                           with i + rot/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * freq[i];
//                           the angle is computed and reduced to [-pi, pi] in double precision, its sine
//                           and cosine in fp32.
//   mi_qk_norm_rope_store   queries and keys get an RMS norm over the head with one gain shared by the heads
//                           (optional; before it an fp32 bias per packed column may be added to q, k and v),
//                           then the rotation of the half layout on their first `rot` dimensions
//                           (angles as above), then a factor each (q_scale, k_scale); both are written back
//                           in place and k goes to its cache page.  The values (optional: v_off < 0 means the
//                           mixer has none here) may be blended with another layer's values of the same
//                           tokens, v <- (1 - lam) v + lam v_other with lam read from device memory; they are
//                           written back in place as well (a later layer may ask for them) and go to the
//                           value pages.  Without pages nothing is stored: a mixer that keeps a state instead
//                           of keys uses the kernel for the rotation alone.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define QK_MAX_PER_LANE 8   // a lane keeps d / 32 values of a head (d <= 256)

template <typename T>
__global__ void __launch_bounds__(128)
qk_bias_norm_store_kernel(T* __restrict__ packed, int stride, int q_off, int k_off, int v_off, int nq, int nkv, int d,
                          int dv, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                          const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                          int values_are_keys, const int* __restrict__ slots, T* __restrict__ kcache,
                          T* __restrict__ vcache, int page_size, int writes) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  T* row = packed + (size_t)t * stride;
  constexpr int EPC = 16 / (int)sizeof(T);
  const int slot = writes ? slots[t] : 0;
  const int page = slot / page_size, offset = slot - page * page_size;
  const int mk = mi_swizzle_mask_rows(d, (int)sizeof(T)), mv = mi_swizzle_mask_rows(dv, (int)sizeof(T));
  const int n_heads = nq + nkv + (values_are_keys ? 0 : nkv);
  // a block's warps take the heads blockIdx.y * warps .. : all heads of a token at once
  for (int h = blockIdx.y * nwarps + warp; h < n_heads; h += gridDim.y * nwarps) {
    if (h >= nq + nkv) {              // values with columns of their own
      if (!writes) continue;
      const int kvh = h - nq - nkv;
      const T* src = row + v_off + kvh * dv;
      T* dst = vcache + ((size_t)(page * nkv + kvh) * page_size + offset) * dv;
      for (int k = lane; k < dv; k += 32) dst[mi_swizzled(k, offset, mv, EPC)] = src[k];
      continue;
    }
    const bool is_q = h < nq;
    const int hh = is_q ? h : h - nq;
    T* x = row + (is_q ? q_off : k_off) + hh * d;
    const float* bias = is_q ? q_bias : k_bias;
    const float* gain = is_q ? q_gain : k_gain;
    float val[QK_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < QK_MAX_PER_LANE; ++j) {
      const int k = lane + 32 * j;
      val[j] = 0.f;
      if (k < d) {
        val[j] = mi_to_float(x[k]) + (bias ? bias[hh * d + k] : 0.f);
        ss += val[j] * val[j];
      }
    }
    T* kdst = nullptr;
    if (!is_q && writes) {
      kdst = kcache + ((size_t)(page * nkv + hh) * page_size + offset) * d;
      if (values_are_keys) {          // the value is the key as projected: before the norm
        T* vdst = vcache + ((size_t)(page * nkv + hh) * page_size + offset) * d;
#pragma unroll
        for (int j = 0; j < QK_MAX_PER_LANE; ++j) {
          const int k = lane + 32 * j;
          if (k < d) vdst[mi_swizzled(k, offset, mk, EPC)] = mi_from_float<T>(val[j]);
        }
      }
    }
    float mult = 1.f;
    if (gain) {
      ss = mi_warp_sum(ss);
      mult = 1.f / sqrtf(ss / (float)d + eps);
    }
#pragma unroll
    for (int j = 0; j < QK_MAX_PER_LANE; ++j) {
      const int k = lane + 32 * j;
      if (k < d) {
        const T y = mi_from_float<T>(gain ? val[j] * mult * gain[k] : val[j]);
        x[k] = y;
        if (kdst) kdst[mi_swizzled(k, offset, mk, EPC)] = y;
      }
    }
  }
}

extern "C" int mi_qk_bias_norm_store(void* packed, int stride, int q_off, int k_off, int v_off, int M, int nq, int nkv,
                                     int d, int dv, const float* q_bias, const float* k_bias, const float* q_gain,
                                     const float* k_gain, float eps, int values_are_keys, const int* slots,
                                     void* kcache, void* vcache, int page_size, int writes, int dtype,
                                     cudaStream_t stream) {
  if (M <= 0) return 0;
  if (d <= 0 || d > 32 * QK_MAX_PER_LANE || dv <= 0) MI_REFUSE("qk_prepare: head size %d must lie in [1, %d]", d, 32 * QK_MAX_PER_LANE);
  if (values_are_keys && dv != d) MI_REFUSE("qk_prepare: values that are the keys have the keys' size, not %d", dv);
  if (writes && (!slots || !kcache || !vcache || page_size <= 0)) MI_REFUSE("qk_prepare: a cache write needs slots and pages");
  const int n_heads = nq + nkv + (values_are_keys ? 0 : nkv);
  const dim3 grid((unsigned)M, (unsigned)((n_heads + 3) / 4 < 64 ? (n_heads + 3) / 4 : 64));
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((qk_bias_norm_store_kernel<float>), grid, 128, 0, stream, (float*)packed, stride, q_off, k_off, v_off, nq, nkv,
              d, dv, q_bias, k_bias, q_gain, k_gain, eps, values_are_keys, slots, (float*)kcache, (float*)vcache,
              page_size, writes);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((qk_bias_norm_store_kernel<bf16>), grid, 128, 0, stream, (bf16*)packed, stride, q_off, k_off, v_off, nq, nkv,
              d, dv, q_bias, k_bias, q_gain, k_gain, eps, values_are_keys, slots, (bf16*)kcache, (bf16*)vcache,
              page_size, writes);
  else
    MI_REFUSE("qk_prepare: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

#define LATENT_MAX_ROT 512

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ packed, int stride, int q_off, int nq, int q_head, int q_rot_off, int c_off,
                      int rank, int rot_dim, int rot, const int* __restrict__ positions,
                      const double* __restrict__ freq, const float* __restrict__ c_gain, float eps,
                      T* __restrict__ qfull, int qfull_stride, int qfull_head, const int* __restrict__ slots,
                      T* __restrict__ kcache, int page_size, int writes) {
  mi_pdl_enter();
  __shared__ float sn[LATENT_MAX_ROT / 2], cs[LATENT_MAX_ROT / 2];
  __shared__ float red[32];
  const int t = blockIdx.x, tid = threadIdx.x;
  const T* row = packed + (size_t)t * stride;
  const int half = rot >> 1;
  const double pos = (double)positions[t];
  for (int i = tid; i < half; i += blockDim.x) {
    // the angle in double precision, brought into [-pi, pi] there; its sine and cosine in fp32
    double a = pos * freq[i];
    a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
    float s, c;
    sincosf((float)a, &s, &c);
    sn[i] = s;
    cs[i] = c;
  }
  // the latent's sum of squares (fixed order: by thread, then by warp)
  float ss = 0.f;
  for (int k = tid; k < rank; k += blockDim.x) {
    const float v = mi_to_float(row[c_off + k]);
    ss += v * v;
  }
  const float mult = 1.f / sqrtf(mi_block_sum(ss, red) / (float)rank + eps);   // its barriers also publish sn, cs
  constexpr int EPC = 16 / (int)sizeof(T);
  const int dk = rank + rot_dim;
  if (writes) {
    const int slot = slots[t];
    const int page = slot / page_size, offset = slot - page * page_size;
    const int mk = mi_swizzle_mask_rows(dk, (int)sizeof(T));
    T* kdst = kcache + ((size_t)page * page_size + offset) * dk;
    for (int k = tid; k < rank; k += blockDim.x)
      kdst[mi_swizzled(k, offset, mk, EPC)] = mi_from_float<T>(mi_to_float(row[c_off + k]) * mult * c_gain[k]);
    const T* kr = row + c_off + rank;
    for (int k = tid; k < rot_dim; k += blockDim.x) {
      float y = mi_to_float(kr[k]);
      if (k < rot) {
        const int i = k < half ? k : k - half;
        const float u = mi_to_float(kr[i]), v = mi_to_float(kr[i + half]);
        float y1, y2;
        mi_rotate(u, v, sn[i], cs[i], y1, y2);
        y = k < half ? y1 : y2;
      }
      kdst[mi_swizzled(rank + k, offset, mk, EPC)] = mi_from_float<T>(y);
    }
  }
  for (int idx = tid; idx < nq * rot_dim; idx += blockDim.x) {
    const int h = idx / rot_dim, k = idx - h * rot_dim;
    const T* qr = row + q_off + h * q_head + q_rot_off;
    float y = mi_to_float(qr[k]);
    if (k < rot) {
      const int i = k < half ? k : k - half;
      const float u = mi_to_float(qr[i]), v = mi_to_float(qr[i + half]);
      float y1, y2;
      mi_rotate(u, v, sn[i], cs[i], y1, y2);
      y = k < half ? y1 : y2;
    }
    qfull[(size_t)t * qfull_stride + h * qfull_head + rank + k] = mi_from_float<T>(y);
  }
}

extern "C" int mi_latent_prepare(const void* packed, int stride, int q_off, int M, int nq, int q_head, int q_rot_off,
                                 int c_off, int rank, int rot_dim, int rot, const int* positions, const double* freq,
                                 const float* c_gain, float eps, void* qfull, int qfull_stride, int qfull_head,
                                 const int* slots, void* kcache, int page_size, int writes, int dtype,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  if (rank <= 0 || rot_dim < 0 || nq <= 0) MI_REFUSE("latent_prepare: bad sizes rank=%d rot_dim=%d heads=%d", rank, rot_dim, nq);
  if (rot < 0 || rot > rot_dim || (rot & 1) || rot > LATENT_MAX_ROT)
    MI_REFUSE("latent_prepare: %d rotated dimensions of %d (an even number up to %d)", rot, rot_dim, LATENT_MAX_ROT);
  if (q_rot_off + rot_dim > q_head || qfull_head < rank + rot_dim) MI_REFUSE("latent_prepare: a head's rotated part lies outside the head");
  if (!positions || (rot > 0 && !freq) || !c_gain || !qfull) MI_REFUSE("latent_prepare: positions, frequencies, gain and qfull are needed");
  if (writes && (!slots || !kcache || page_size <= 0)) MI_REFUSE("latent_prepare: a cache write needs slots and pages");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((latent_prepare_kernel<float>), M, 128, 0, stream, (const float*)packed, stride, q_off, nq, q_head, q_rot_off,
              c_off, rank, rot_dim, rot, positions, freq, c_gain, eps, (float*)qfull, qfull_stride, qfull_head, slots,
              (float*)kcache, page_size, writes);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((latent_prepare_kernel<bf16>), M, 128, 0, stream, (const bf16*)packed, stride, q_off, nq, q_head, q_rot_off,
              c_off, rank, rot_dim, rot, positions, freq, c_gain, eps, (bf16*)qfull, qfull_stride, qfull_head, slots,
              (bf16*)kcache, page_size, writes);
  else
    MI_REFUSE("latent_prepare: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}


#define ROPE_MAX_D 1024

template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_rope_store_kernel(T* __restrict__ packed, int stride, int q_off, int k_off, int v_off, int nq, int nkv, int d,
                          int dv, const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                          int rot, const int* __restrict__ positions, const double* __restrict__ freq, float q_scale,
                          float k_scale, const T* __restrict__ v_other, int v_other_stride,
                          const float* __restrict__ lam_ptr, const int* __restrict__ slots, T* __restrict__ kcache,
                          T* __restrict__ vcache, int page_size, int writes, float* __restrict__ qk_out,
                          int qk_out_stride, const float* __restrict__ bias) {
  // bias [stride]: added (fp32) to the q, k and v columns before anything else, by packed column.
  // qk_out [M, (nq + nkv) * d] fp32: the finished queries and keys go there unrounded (for a recurrence
  // that reads them in fp32) and the packed rows keep what the projection left.
  mi_pdl_enter();
  extern __shared__ float rope_sm[];
  const int half = rot >> 1;
  float* sn = rope_sm;                 // [half]
  float* cs = sn + half;               // [half]
  float* buf = cs + half;              // [warps][d] a head's values after the norm
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (half > 0) {
    const double pos = (double)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      double a = pos * freq[i];
      a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
      float s, c;
      sincosf((float)a, &s, &c);
      sn[i] = s;
      cs[i] = c;
    }
  }
  __syncthreads();
  T* row = packed + (size_t)t * stride;
  constexpr int EPC = 16 / (int)sizeof(T);
  const int slot = writes ? slots[t] : 0;
  const int page = slot / page_size, offset = slot - page * page_size;
  const int mk = mi_swizzle_mask_rows(d, (int)sizeof(T)), mv = mi_swizzle_mask_rows(dv, (int)sizeof(T));
  const int n_v = v_off >= 0 ? nkv : 0;
  const float lam = lam_ptr ? *lam_ptr : 0.f;
  float* mine = buf + (size_t)warp * d;
  for (int h = blockIdx.y * nwarps + warp; h < nq + nkv + n_v; h += gridDim.y * nwarps) {
    if (h >= nq + nkv) {               // values
      const int kvh = h - nq - nkv;
      T* src = row + v_off + kvh * dv;
      T* dst = writes ? vcache + ((size_t)(page * nkv + kvh) * page_size + offset) * dv : nullptr;
      const T* other = v_other ? v_other + (size_t)t * v_other_stride + kvh * dv : nullptr;
      for (int k = lane; k < dv; k += 32) {
        T y = src[k];
        if (bias) {
          y = mi_from_float<T>(mi_to_float(y) + bias[v_off + kvh * dv + k]);
          if (!other) src[k] = y;
        }
        if (other) {
          y = mi_from_float<T>((1.f - lam) * mi_to_float(y) + lam * mi_to_float(other[k]));
          src[k] = y;
        }
        if (dst) dst[mi_swizzled(k, offset, mv, EPC)] = y;
      }
      continue;
    }
    const bool is_q = h < nq;
    const int hh = is_q ? h : h - nq;
    T* x = row + (is_q ? q_off : k_off) + hh * d;
    const float* gain = is_q ? q_gain : k_gain;
    const float post = is_q ? q_scale : k_scale;
    float ss = 0.f;
    const float* xb = bias ? bias + (is_q ? q_off : k_off) + hh * d : nullptr;
    for (int k = lane; k < d; k += 32) {
      const float v = mi_to_float(x[k]) + (xb ? xb[k] : 0.f);
      mine[k] = v;
      ss += v * v;
    }
    if (gain) {
      ss = mi_warp_sum(ss);
      const float mult = 1.f / sqrtf(ss / (float)d + eps);
      for (int k = lane; k < d; k += 32) mine[k] = mine[k] * mult * gain[k];
    }
    __syncwarp();
    T* kdst = (!is_q && writes) ? kcache + ((size_t)(page * nkv + hh) * page_size + offset) * d : nullptr;
    for (int k = lane; k < d; k += 32) {
      float y = mine[k];
      if (k < rot) {
        const int i = k < half ? k : k - half;
        float y1, y2;
        mi_rotate(mine[i], mine[i + half], sn[i], cs[i], y1, y2);
        y = k < half ? y1 : y2;
      }
      const T out = mi_from_float<T>(y * post);
      if (qk_out) qk_out[(size_t)t * qk_out_stride + (size_t)h * d + k] = y * post;
      else x[k] = out;
      if (kdst) kdst[mi_swizzled(k, offset, mk, EPC)] = out;
    }
    __syncwarp();                      // the warp's buffer is free for its next head
  }
}

extern "C" int mi_qk_norm_rope_store(void* packed, int stride, int q_off, int k_off, int v_off, int M, int nq, int nkv,
                                     int d, int dv, const float* q_gain, const float* k_gain, float eps, int rot,
                                     const int* positions, const double* freq, float q_scale, float k_scale,
                                     const void* v_other, int v_other_stride, const float* lam, const int* slots,
                                     void* kcache, void* vcache, int page_size, int writes, float* qk_out,
                                     int qk_out_stride, const float* bias, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (qk_out && qk_out_stride < (nq + nkv) * d) MI_REFUSE("qk_prepare: fp32 rows of %d for %d heads of %d", qk_out_stride, nq + nkv, d);
  if (d <= 0 || d > ROPE_MAX_D || dv < 0) MI_REFUSE("qk_prepare: head size %d must lie in [1, %d]", d, ROPE_MAX_D);
  if (rot < 0 || rot > d || (rot & 1)) MI_REFUSE("qk_prepare: %d rotated dimensions of %d", rot, d);
  if (rot > 0 && (!positions || !freq)) MI_REFUSE("qk_prepare: a rotation needs positions and frequencies");
  if (v_other && !lam) MI_REFUSE("qk_prepare: blending values needs the blend's weight");
  if (writes && (!slots || !kcache || page_size <= 0 || (v_off >= 0 && !vcache)))
    MI_REFUSE("qk_prepare: a cache write needs slots and pages");
  const int n_heads = nq + nkv + (v_off >= 0 ? nkv : 0);
  const dim3 grid((unsigned)M, (unsigned)((n_heads + 3) / 4 < 64 ? (n_heads + 3) / 4 : 64));
  const size_t smem = ((size_t)rot + 4 * (size_t)d) * sizeof(float);
#define MI_GO(T)                                                                                                       \
  MI_LAUNCH((qk_norm_rope_store_kernel<T>), grid, 128, smem, stream, (T*)packed, stride, q_off, k_off, v_off, nq, nkv, \
            d, dv, q_gain, k_gain, eps, rot, positions, freq, q_scale, k_scale, (const T*)v_other, v_other_stride,    \
            lam, slots, (T*)kcache, (T*)vcache, page_size, writes, qk_out, qk_out_stride, bias)
  if (dtype == MI_DTYPE_F32) MI_GO(float);
  else if (dtype == MI_DTYPE_BF16) MI_GO(bf16);
  else MI_REFUSE("qk_prepare: unknown dtype %d", dtype);
#undef MI_GO
  MI_RETURN_LAUNCH_STATUS();
}
