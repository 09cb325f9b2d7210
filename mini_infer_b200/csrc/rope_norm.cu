// What stands around an attention whose queries and keys are rotated in the interleaved layout
// and then brought to unit root mean square, and whose heads are gated before the output
// projection.
//
//   mi_rope_norm_store   for every token and head: q and k are rotated on their first `rot` dimensions
//                        (dimension 2i pairs with 2i+1; the pair (u, v) at position p becomes
//                        (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i]), then, with
//                        unit_norm, divided by sqrt(mean(x^2) + eps) over the head; q is written back
//                        in place, k and v go to their cache pages (k of size d, v of size dv).
//                        Angles, sines, cosines and the norm are fp32; each value is rounded once.
//   mi_gate_mul          out[t, c] = T(x[t, c] * act(g[t, c / per]) * scale), act = sigmoid or SiLU; per = 1: a
//                        gate per element, per = a head's size: one gate per head.
//
// q, k, v and the gate are column ranges of one packed projection [tokens, stride].
#include "common.cuh"

MI_DEFINE_ERROR_API()

template <typename T>
__global__ void __launch_bounds__(128)
rope_norm_store_kernel(T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off,
                       const int* __restrict__ positions, const float* __restrict__ inv_freq,
                       const int* __restrict__ slots, T* __restrict__ kcache, T* __restrict__ vcache,
                       int nq, int nkv, int d, int dv, int rot, int unit_norm, float eps, int page_size,
                       int writes) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float pos = positions ? (float)positions[t] : 0.f;
  T* row = qkv + (size_t)t * stride;
  constexpr int EPC = 16 / (int)sizeof(T);
  const int slot = writes ? slots[t] : 0;
  const int page = slot / page_size, offset = slot - page * page_size;
  const int mk = mi_swizzle_mask_rows(d, (int)sizeof(T)), mv = mi_swizzle_mask_rows(dv, (int)sizeof(T));
  const int npairs = (d + 1) >> 1;
  // heads 0..nq-1: queries; nq..nq+nkv-1: keys; then the values
  for (int h = warp; h < nq + 2 * nkv; h += nwarps) {
    if (h >= nq + nkv) {
      if (!writes) continue;
      const int kvh = h - nq - nkv;
      const T* src = row + v_off + kvh * dv;
      T* dst = vcache + ((size_t)(page * nkv + kvh) * page_size + offset) * dv;
      for (int k = lane; k < dv; k += 32) dst[mi_swizzled(k, offset, mv, EPC)] = src[k];
      continue;
    }
    const bool is_q = h < nq;
    T* x = is_q ? row + q_off + h * d : row + k_off + (h - nq) * d;
    if (!is_q && !writes && !unit_norm && rot == 0) continue;
    float ss = 0.f;
    // a lane keeps at most 4 pairs (d <= 256)
    float a0[4], a1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = lane + 32 * j;
      a0[j] = a1[j] = 0.f;
      if (p < npairs) {
        float u = mi_to_float(x[2 * p]);
        float v = (2 * p + 1 < d) ? mi_to_float(x[2 * p + 1]) : 0.f;
        if (2 * p + 1 < rot) {
          float s, c;
          sincosf(pos * inv_freq[p], &s, &c);
          float ru, rv;
          mi_rotate(u, v, s, c, ru, rv);
          u = ru;
          v = rv;
        }
        a0[j] = u;
        a1[j] = v;
        ss += u * u + v * v;
      }
    }
    float mult = 1.f;
    if (unit_norm) {
      ss = mi_warp_sum(ss);
      mult = 1.f / sqrtf(ss / (float)d + eps);
    }
    T* kdst = nullptr;
    if (!is_q && writes) kdst = kcache + ((size_t)(page * nkv + (h - nq)) * page_size + offset) * d;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = lane + 32 * j;
      if (p < npairs) {
        const T u = mi_from_float<T>(a0[j] * mult), v = mi_from_float<T>(a1[j] * mult);
        x[2 * p] = u;
        if (2 * p + 1 < d) x[2 * p + 1] = v;
        if (kdst) {
          kdst[mi_swizzled(2 * p, offset, mk, EPC)] = u;
          if (2 * p + 1 < d) kdst[mi_swizzled(2 * p + 1, offset, mk, EPC)] = v;
        }
      }
    }
  }
}

extern "C" int mi_rope_norm_store(void* qkv, int stride, int q_off, int k_off, int v_off, const int* positions,
                                  const float* inv_freq, const int* slots, void* kcache, void* vcache, int M,
                                  int nq, int nkv, int d, int dv, int rot, int unit_norm, float eps,
                                  int page_size, int writes, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (d <= 0 || d > 256 || dv <= 0 || dv > 256) MI_REFUSE("rope_norm: head sizes %d and %d must lie in [1, 256]", d, dv);
  if (rot < 0 || rot > d || (rot & 1)) MI_REFUSE("rope_norm: %d rotated dimensions of %d", rot, d);
  if (writes && (!slots || !kcache || !vcache || page_size <= 0)) MI_REFUSE("rope_norm: a cache write needs slots and pages");
  if (rot > 0 && (!positions || !inv_freq)) MI_REFUSE("rope_norm: a rotation needs positions and frequencies");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((rope_norm_store_kernel<float>), M, 128, 0, stream, (float*)qkv, stride, q_off, k_off, v_off, positions,
              inv_freq, slots, (float*)kcache, (float*)vcache, nq, nkv, d, dv, rot, unit_norm, eps, page_size, writes);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((rope_norm_store_kernel<bf16>), M, 128, 0, stream, (bf16*)qkv, stride, q_off, k_off, v_off, positions,
              inv_freq, slots, (bf16*)kcache, (bf16*)vcache, nq, nkv, d, dv, rot, unit_norm, eps, page_size, writes);
  else
    MI_REFUSE("rope_norm: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// act: 1 sigmoid, 2 SiLU
template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ g, int g_stride,
                                T* __restrict__ out, int out_stride, int M, int C, int act, float scale, int per) {
  mi_pdl_enter();
  const size_t n = (size_t)M * C;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / C), c = (int)(idx - (size_t)t * C);
    float a = 1.f;                       // act 0: no gate, the factor alone
    if (act) {
      const float gv = mi_to_float(g[(size_t)t * g_stride + c / per]);
      const float sg = 1.f / (1.f + expf(-gv));
      a = act == 2 ? gv * sg : sg;
    }
    out[(size_t)t * out_stride + c] = mi_from_float<T>(mi_to_float(x[(size_t)t * x_stride + c]) * a * scale);
  }
}

extern "C" int mi_gate_mul(const void* x, int x_stride, const void* g, int g_stride, void* out, int out_stride,
                           int M, int C, int act, float scale, int per, int dtype, cudaStream_t stream) {
  if (M <= 0 || C <= 0) return 0;
  if (per <= 0) MI_REFUSE("gate_mul: %d columns per gate", per);
  if (act < 0 || act > 2 || (act && !g)) MI_REFUSE("gate_mul: unknown activation %d, or no gate for it", act);
  const size_t n = (size_t)M * C;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((gate_mul_kernel<float>), blocks, 256, 0, stream, (const float*)x, x_stride, (const float*)g, g_stride,
              (float*)out, out_stride, M, C, act, scale, per);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((gate_mul_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)x, x_stride, (const bf16*)g, g_stride,
              (bf16*)out, out_stride, M, C, act, scale, per);
  else
    MI_REFUSE("gate_mul: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}
