// Routed experts: every token goes through the `top` experts its router picks.
//
//   mi_moe_select     from the router logits z = W_r x (fp32, a matrix product): the `top` largest of a token
//                     (ties: the lower index; optionally among the experts of the best groups only) and
//                     their weights (the softmax over those alone, or their share of the softmax over all
//                     experts, times a factor, or their sigmoids times a factor, chosen with a correction
//                     added per expert) -> ids [M, top] int32, weights [M, top] fp32
//   mi_moe_plan       sorts the M*top (token, choice) entries by expert: perm[pos] = entry, inv[entry] =
//                     pos, offsets[E + 1], and the list of row tiles (expert, first row, rows) that the
//                     grouped products walk.  Nothing comes back to the host: the products are launched
//                     for the largest possible number of tiles and the surplus blocks leave at once.
//                     Tiles have 64 rows, or 8 for steps that bring an expert only a few rows.
//   mi_moe_gate_up    act[pos, :] = glu(W_gate[e] x_token, W_up[e] x_token) for the entries of each expert
//   mi_moe_down       y[pos, :] = W_down[e] act[pos, :]   (fp32)
//   mi_moe_gather     xs[pos, :] = x[token of pos, :], for steps whose products are a library's grouped product
//   mi_moe_combine    out[t, :] = T(sum_k weight[t, k] * y[inv[t*top + k], :] + shared[t, :]), the shared
//                     expert's row optionally times sigmoid(gate[t])
//   mi_clamped_glu    the same activation for a dense expert: out = glu(gu[:, :I], gu[:, I:])
//
// glu(g, u) = g' * sigmoid(alpha * g') * (u' + offset), g' = min(g, limit), u' = clamp(u, -limit, limit).
// An infinite limit with alpha = 1 and offset = 0 is the plain silu(g) * u.
//
// Three products live here, all with fp32 accumulation, and none lets a row's result depend on which
// other rows share its tile: float32 on CUDA cores, k ascending (moe_gemm_kernel); bfloat16 tiles of 64
// rows on the tensor cores (mma.sync m16n8k16, moe_gemm_mma_kernel); bfloat16 tiles of 8 rows that
// stream an expert's weights, one warp per output column (moe_stream_kernel).  Large bfloat16 steps
// whose rows are whole 16-byte pieces go to the library's grouped product instead (the caller gathers
// the rows with mi_moe_gather and passes the experts' row ranges from the plan).
#include "common.cuh"

MI_DEFINE_ERROR_API()

__device__ __forceinline__ float mi_clamped_glu_value(float g, float u, float limit, float alpha, float offset) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + offset);
}

// ------------------------------------------------------------------------------------------ router
// The logits [M, E] (fp32) come from a matrix product; one warp per token picks the `top` largest
// choice scores (ties: the lower index).  Three ways to score and weigh.  mode 0: the choice score is
// the logit, the weights the softmax over the chosen logits alone.  mode 1: scores are the softmax over all
// experts (the logit orders alike); the chosen experts' scores are divided by their sum (+ 1e-20) and
// multiplied by `scale`.  mode 2: scores are sigmoid(logit), the choice score adds `correction[e]` (may be
// absent), the weights are the chosen experts' scores times `scale` (no division by their sum).  With n_groups > 1
// the experts lie in n_groups equal groups of neighbours and only experts of the `keep` best groups (ties:
// the lower index) can be chosen; a group counts as its best choice score (group_top2 = 0) or as the sum
// of its two best (group_top2 = 1).
#define ROUTE_MAX_PER_LANE 8
#define ROUTE_WARPS 4

__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_select_kernel(const float* __restrict__ logits, int stride, int* __restrict__ ids,
                  float* __restrict__ weights, int M, int E, int top, int mode, int n_groups,
                  int keep, float scale, const float* __restrict__ correction, int group_top2) {
  mi_pdl_enter();
  __shared__ float choice_sh[ROUTE_WARPS][32 * ROUTE_MAX_PER_LANE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= M) return;
  const float* z = logits + (size_t)t * stride;
  float lg[ROUTE_MAX_PER_LANE];       // choice scores; minus infinity: out of the race
  float sc[ROUTE_MAX_PER_LANE];       // mode 2: the scores that become weights
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    lg[i] = e < E ? z[e] : -INFINITY;
    sc[i] = 0.f;
    if (mode == 2 && e < E) {
      sc[i] = 1.f / (1.f + expf(-lg[i]));
      lg[i] = sc[i] + (correction ? correction[e] : 0.f);
    }
  }
  float zmax = -INFINITY, zsum = 0.f;
  if (mode == 1) {
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) zmax = fmaxf(zmax, lg[i]);
    zmax = mi_warp_max(zmax);
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (lane + 32 * i < E) zsum += expf(lg[i] - zmax);
    zsum = mi_warp_sum(zsum);
  }
  if (n_groups > 1) {
    // group g's score sits with lane g % 32, place g / 32; the groups that stay: `keep` times the
    // best group that is still in; experts of the others are taken out
    const int per = E / n_groups;
    float* mine = choice_sh[warp];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (lane + 32 * i < E) mine[lane + 32 * i] = lg[i];
    __syncwarp();
    float gs[ROUTE_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int g = lane + 32 * i;
      gs[i] = -INFINITY;
      if (g < n_groups) {
        float b1 = -INFINITY, b2 = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = mine[e];
          if (v > b1) { b2 = b1; b1 = v; }
          else if (v > b2) b2 = v;
        }
        gs[i] = (group_top2 && per > 1) ? b1 + b2 : b1;
      }
    }
    unsigned kept_mask = 0u;             // bit i: this lane's group lane + 32 i stays
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
        const int g = lane + 32 * i;
        if (g < n_groups && !((kept_mask >> i) & 1u) && (gs[i] > best || (gs[i] == best && g < best_g))) {
          best = gs[i];
          best_g = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ob > best || (ob == best && og < best_g)) {
          best = ob;
          best_g = og;
        }
      }
      if (best_g == 0x7fffffff) break;
      if ((best_g & 31) == lane) kept_mask |= 1u << (best_g >> 5);
    }
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      const int g = e < E ? e / per : 0;
      const unsigned owner_mask = __shfl_sync(0xffffffffu, kept_mask, g & 31);   // every lane takes part
      if (e < E && !((owner_mask >> (g >> 5)) & 1u)) lg[i] = -INFINITY;
    }
  }
  float my_val = 0.f, denom = 0.f, first = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (lg[i] > best || (lg[i] == best && e < best_e)) && lg[i] != -INFINITY) {
        best = lg[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    float score = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (best_e == lane + 32 * i) {
        lg[i] = -INFINITY;   // taken
        score = sc[i];
      }
    if (k == 0) first = best;
    float p;
    if (mode == 2) p = __shfl_sync(0xffffffffu, score, best_e & 31);
    else p = mode == 1 ? expf(best - zmax) / zsum : expf(best - first);
    denom += p;
    if (lane == k) {
      my_val = p;
      my_id = best_e;
    }
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = my_id;
    weights[(size_t)t * top + lane] = mode == 2 ? my_val * scale
                                    : mode == 1 ? my_val / (denom + 1e-20f) * scale : my_val / denom;
  }
}

extern "C" int mi_moe_select(const float* logits, int stride, int* ids, float* weights, int M, int E, int top,
                             int mode, int n_groups, int keep, float scale, const float* correction,
                             int group_top2, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > 32 * ROUTE_MAX_PER_LANE) MI_REFUSE("moe: %d experts (1 to %d are taken)", E, 32 * ROUTE_MAX_PER_LANE);
  if (top <= 0 || top > E || top > 32) MI_REFUSE("moe: %d of %d experts per token", top, E);
  if (mode < 0 || mode > 2) MI_REFUSE("moe: unknown way %d to score the experts", mode);
  if (n_groups > 1) {
    if (E % n_groups) MI_REFUSE("moe: %d experts are no %d equal groups", E, n_groups);
    if (keep <= 0 || keep > n_groups) MI_REFUSE("moe: %d of %d groups kept", keep, n_groups);
    if (keep * (E / n_groups) < top) MI_REFUSE("moe: %d groups of %d experts cannot give %d experts", keep, E / n_groups, top);
  }
  MI_LAUNCH((moe_select_kernel), (M + ROUTE_WARPS - 1) / ROUTE_WARPS, 32 * ROUTE_WARPS, 0, stream, logits, stride, ids,
            weights, M, E, top, mode, n_groups, keep, scale, correction, group_top2);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ plan
#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

// plan layout (int32): [0] number of tiles, [1 .. E+1] offsets, then 3 ints per tile (expert, first row, rows)
__global__ void moe_plan_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ perm,
                                int* __restrict__ inv, int* __restrict__ plan, int tile_rows) {
  mi_pdl_enter();
  extern __shared__ int sh[];
  int* counts = sh;            // [E]
  int* cursor = sh + E;        // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int* offsets = plan + 1;
    int* tiles = plan + 2 + E;
    int run = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      const int end = run + counts[e];
      for (int r0 = run; r0 < end; r0 += tile_rows) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = r0;
        tiles[3 * nt + 2] = min(tile_rows, end - r0);
        ++nt;
      }
      run = end;
    }
    offsets[E] = run;
    plan[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int pos = atomicAdd(&cursor[ids[i]], 1);
    perm[pos] = i;
    inv[i] = pos;
  }
}

#define FEW_ROWS 8
// rows per tile: TILE_M for the tiled products, FEW_ROWS for the streaming ones (few rows per expert)
extern "C" int mi_moe_tile_rows(int few) { return few ? FEW_ROWS : TILE_M; }

extern "C" int mi_moe_plan(const int* ids, int n, int E, int* perm, int* inv, int* plan, int tile_rows,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > 4096) MI_REFUSE("moe: %d experts", E);
  if (tile_rows != TILE_M && tile_rows != FEW_ROWS) MI_REFUSE("moe: tiles of %d rows", tile_rows);
  MI_LAUNCH((moe_plan_kernel), 1, 1024, 2 * E * sizeof(int), stream, ids, n, E, perm, inv, plan, tile_rows);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ grouped products
// A tile is TILE_M rows of one expert times TILE_N output columns; 256 threads, 4 x 4 outputs each.
// GATED: A rows are gathered (token = perm[pos] / top), two weight matrices, the activation in the
// epilogue, output in T.  Otherwise A rows are the sorted rows themselves and the output is fp32.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w0, const T* __restrict__ w1,
                long long w_expert_stride, const int* __restrict__ perm, int top, const int* __restrict__ plan,
                int E, void* __restrict__ out_, int N, int K, float limit, float alpha, float offset) {
  mi_pdl_enter();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* td = plan + 2 + E + 3 * tile;
  const int e = td[0], row0 = td[1], rows = td[2];
  const int n0 = blockIdx.x * TILE_N;
  __shared__ float As[TILE_K][TILE_M + 4];
  __shared__ float B0[TILE_K][TILE_N + 4];
  __shared__ float B1[GATED ? TILE_K : 1][TILE_N + 4];
  __shared__ int arow[TILE_M];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < TILE_M) {
    int r = -1;
    if (tid < rows) r = GATED ? perm[row0 + tid] / top : row0 + tid;
    arow[tid] = r;
  }
  const T* wb0 = w0 + (size_t)e * w_expert_stride;
  const T* wb1 = GATED ? w1 + (size_t)e * w_expert_stride : nullptr;
  float acc0[4][4], acc1[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.f;
  __syncthreads();
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    // 64 x 16 elements of each operand: 4 per thread, k fastest
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;
      const int r = idx >> 4, kk = idx & 15;
      const int kg = k0 + kk;
      const int ar = arow[r];
      As[kk][r] = (ar >= 0 && kg < K) ? mi_to_float(a[(size_t)ar * a_stride + kg]) : 0.f;
      const int n = n0 + r;
      const bool ok = n < N && kg < K;
      B0[kk][r] = ok ? mi_to_float(wb0[(size_t)n * K + kg]) : 0.f;
      if (GATED) B1[kk][r] = ok ? mi_to_float(wb1[(size_t)n * K + kg]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float av[4], b0[4], b1[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b0[j] = B0[kk][tx * 4 + j];
        if (GATED) b1[j] = B1[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc0[i][j] = fmaf(av[i], b0[j], acc0[i][j]);
          if (GATED) acc1[i][j] = fmaf(av[i], b1[j], acc1[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (GATED)
        reinterpret_cast<T*>(out_)[(size_t)(row0 + r) * N + n] =
            mi_from_float<T>(mi_clamped_glu_value(acc0[i][j], acc1[i][j], limit, alpha, offset));
      else
        reinterpret_cast<float*>(out_)[(size_t)(row0 + r) * N + n] = acc0[i][j];
    }
  }
}

// ------------------------------------------------------------------------------------------ the same on tensor cores
// bfloat16 only.  64 rows x 64 columns per block, k in steps of 32; four warps, each 32 x 32 of the
// tile as 2 x 4 mma.m16n8k16 tiles (twice that with two weight matrices).  Operands go through
// shared memory with rows of 40 elements, which makes the fragments' 32-bit reads conflict-free.
// Rows of 8 elements are fetched as one 16-byte load where k and the pointers allow it.
#define MMA_K 32
#define MMA_LD (MMA_K + 8)

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// 64 rows x 32 k of a row-major operand into shared memory; row pointers may be null (zero rows)
__device__ __forceinline__ void mma_stage(bf16 (*dst)[MMA_LD], const bf16* const* rowptr, int k0, int K, bool vec,
                                          int tid) {
  if (vec) {   // 64 rows x 4 chunks of 8 elements: 2 chunks per thread
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = tid + 128 * it;
      const int r = idx >> 2, c8 = (idx & 3) << 3;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      const bf16* src = rowptr[r];
      if (src && k0 + c8 < K) v = *reinterpret_cast<const uint4*>(src + k0 + c8);   // K % 8 == 0: whole chunks
      *reinterpret_cast<uint4*>(&dst[r][c8]) = v;
    }
  } else {
    for (int idx = tid; idx < TILE_M * MMA_K; idx += 128) {
      const int r = idx / MMA_K, kk = idx - r * MMA_K;
      const bf16* src = rowptr[r];
      dst[r][kk] = (src && k0 + kk < K) ? src[k0 + kk] : __float2bfloat16_rn(0.f);
    }
  }
}

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ a, int a_stride, const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                    long long w_expert_stride, const int* __restrict__ perm, int top, const int* __restrict__ plan,
                    int E, void* __restrict__ out_, int N, int K, float limit, float alpha, float offset, int vec) {
  mi_pdl_enter();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* td = plan + 2 + E + 3 * tile;
  const int e = td[0], row0 = td[1], rows = td[2];
  const int n0 = blockIdx.x * TILE_N;
  __shared__ __align__(16) bf16 As[TILE_M][MMA_LD];
  __shared__ __align__(16) bf16 B0[TILE_N][MMA_LD];
  __shared__ __align__(16) bf16 B1[GATED ? TILE_N : 1][MMA_LD];
  __shared__ const bf16* aptr[TILE_M];
  __shared__ const bf16* b0ptr[TILE_N];
  __shared__ const bf16* b1ptr[TILE_N];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
  const bf16* wb0 = w0 + (size_t)e * w_expert_stride;
  const bf16* wb1 = GATED ? w1 + (size_t)e * w_expert_stride : nullptr;
  if (tid < TILE_M) {
    const bf16* p = nullptr;
    if (tid < rows) p = a + (size_t)(GATED ? perm[row0 + tid] / top : row0 + tid) * a_stride;
    aptr[tid] = p;
    const int n = n0 + tid;
    b0ptr[tid] = n < N ? wb0 + (size_t)n * K : nullptr;
    b1ptr[tid] = (GATED && n < N) ? wb1 + (size_t)n * K : nullptr;
  }
  float acc0[2][4][4], acc1[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc0[i][j][c] = 0.f;
        if (GATED) acc1[i][j][c] = 0.f;
      }
  __syncthreads();
  for (int k0 = 0; k0 < K; k0 += MMA_K) {
    mma_stage(As, aptr, k0, K, vec != 0, tid);
    mma_stage(B0, b0ptr, k0, K, vec != 0, tid);
    if (GATED) mma_stage(B1, b1ptr, k0, K, vec != 0, tid);
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < MMA_K; ks += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm * 32 + i * 16 + g;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * t + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn * 32 + j * 8 + g;
        uint32_t bf[2];
        bf[0] = *reinterpret_cast<const uint32_t*>(&B0[n][ks + 2 * t]);
        bf[1] = *reinterpret_cast<const uint32_t*>(&B0[n][ks + 2 * t + 8]);
#pragma unroll
        for (int i = 0; i < 2; ++i) mma_bf16(acc0[i][j], af[i], bf);
        if (GATED) {
          bf[0] = *reinterpret_cast<const uint32_t*>(&B1[n][ks + 2 * t]);
          bf[1] = *reinterpret_cast<const uint32_t*>(&B1[n][ks + 2 * t + 8]);
#pragma unroll
          for (int i = 0; i < 2; ++i) mma_bf16(acc1[i][j], af[i], bf);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = wm * 32 + i * 16 + g + (c >> 1) * 8;
        const int n = n0 + wn * 32 + j * 8 + 2 * t + (c & 1);
        if (r >= rows || n >= N) continue;
        if (GATED)
          reinterpret_cast<bf16*>(out_)[(size_t)(row0 + r) * N + n] =
              __float2bfloat16_rn(mi_clamped_glu_value(acc0[i][j][c], acc1[i][j][c], limit, alpha, offset));
        else
          reinterpret_cast<float*>(out_)[(size_t)(row0 + r) * N + n] = acc0[i][j][c];
      }
}

// whether rows of k elements starting at these pointers can be fetched in 16-byte pieces
static int mma_vec_ok(const void* a, long long a_stride, const void* w0, const void* w1, int K) {
  return K % 8 == 0 && a_stride % 8 == 0 && mi_aligned(a, 16) && mi_aligned(w0, 16) && (!w1 || mi_aligned(w1, 16));
}

// ------------------------------------------------------------------------------------------ few rows per expert
// A decode step brings an expert a handful of rows: the product is a stream of that expert's weights.
// Tiles have at most FEW_ROWS rows; a warp owns one output column, its lanes walk k in 16-byte pieces
// (several loads in flight per lane), the tile's rows of x come through the L1, and the lanes' sums
// are added at the end.  bfloat16, k a multiple of 8, 16-byte aligned rows.
__device__ __forceinline__ void fma8(float& acc, const uint4& w, const uint4& x) {
  const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
  const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 wf = __bfloat1622float2(wp[i]), xf = __bfloat1622float2(xp[i]);
    acc = fmaf(wf.x, xf.x, acc);
    acc = fmaf(wf.y, xf.y, acc);
  }
}

template <bool GATED>
__global__ void __launch_bounds__(256)
moe_stream_kernel(const bf16* __restrict__ a, int a_stride, const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                  long long w_expert_stride, const int* __restrict__ perm, int top, const int* __restrict__ plan,
                  int E, void* __restrict__ out_, int N, int K, float limit, float alpha, float offset) {
  mi_pdl_enter();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* td = plan + 2 + E + 3 * tile;
  const int e = td[0], row0 = td[1], rows = td[2];
  __shared__ const bf16* aptr[FEW_ROWS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < FEW_ROWS)
    aptr[tid] = tid < rows ? a + (size_t)(GATED ? perm[row0 + tid] / top : row0 + tid) * a_stride : nullptr;
  __syncthreads();
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const bf16* wr0 = w0 + (size_t)e * w_expert_stride + (size_t)n * K;
  const bf16* wr1 = GATED ? w1 + (size_t)e * w_expert_stride + (size_t)n * K : nullptr;
  float acc0[FEW_ROWS], acc1[FEW_ROWS];
#pragma unroll
  for (int r = 0; r < FEW_ROWS; ++r) acc0[r] = acc1[r] = 0.f;
  // two pieces of every weight row per turn, all four loads in flight before the first is used
  for (int k = lane * 8; k < K; k += 512) {
    const bool two = k + 256 < K;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4 wa0 = *reinterpret_cast<const uint4*>(wr0 + k);
    const uint4 wb0 = two ? *reinterpret_cast<const uint4*>(wr0 + k + 256) : zero;
    const uint4 wa1 = GATED ? *reinterpret_cast<const uint4*>(wr1 + k) : zero;
    const uint4 wb1 = (GATED && two) ? *reinterpret_cast<const uint4*>(wr1 + k + 256) : zero;
#pragma unroll
    for (int r = 0; r < FEW_ROWS; ++r) {
      if (r < rows) {
        const uint4 xa = __ldg(reinterpret_cast<const uint4*>(aptr[r] + k));
        fma8(acc0[r], wa0, xa);
        if (GATED) fma8(acc1[r], wa1, xa);
        if (two) {
          const uint4 xb = __ldg(reinterpret_cast<const uint4*>(aptr[r] + k + 256));
          fma8(acc0[r], wb0, xb);
          if (GATED) fma8(acc1[r], wb1, xb);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < FEW_ROWS; ++r) {
    if (r < rows) {
      const float s0 = mi_warp_sum(acc0[r]);
      const float s1 = GATED ? mi_warp_sum(acc1[r]) : 0.f;
      if (lane == 0) {
        if (GATED)
          reinterpret_cast<bf16*>(out_)[(size_t)(row0 + r) * N + n] =
              __float2bfloat16_rn(mi_clamped_glu_value(s0, s1, limit, alpha, offset));
        else
          reinterpret_cast<float*>(out_)[(size_t)(row0 + r) * N + n] = s0;
      }
    }
  }
}

static int max_tiles(int n_entries, int E, int tile_rows) { return (n_entries + tile_rows - 1) / tile_rows + E; }

extern "C" int mi_moe_gate_up(const void* x, int x_stride, const void* w_gate, const void* w_up,
                              long long w_expert_stride, const int* perm, int top, const int* plan, int E,
                              void* act, int n_entries, int ff, int H, float limit, float alpha, float offset,
                              int tile_rows, int dtype, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (tile_rows == FEW_ROWS) {
    if (dtype != MI_DTYPE_BF16 || !mma_vec_ok(x, x_stride, w_gate, w_up, H))
      MI_REFUSE("moe: the streaming product takes bfloat16 rows of whole 16-byte pieces");
    dim3 g((ff + 7) / 8, max_tiles(n_entries, E, FEW_ROWS));
    if (g.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
    MI_LAUNCH((moe_stream_kernel<true>), g, 256, 0, stream, (const bf16*)x, x_stride, (const bf16*)w_gate,
              (const bf16*)w_up, w_expert_stride, perm, top, plan, E, act, ff, H, limit, alpha, offset);
    MI_RETURN_LAUNCH_STATUS();
  }
  dim3 grid((ff + TILE_N - 1) / TILE_N, max_tiles(n_entries, E, TILE_M));
  if (grid.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_gemm_kernel<float, true>), grid, 256, 0, stream, (const float*)x, x_stride, (const float*)w_gate,
              (const float*)w_up, w_expert_stride, perm, top, plan, E, act, ff, H, limit, alpha, offset);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_gemm_mma_kernel<true>), grid, 128, 0, stream, (const bf16*)x, x_stride, (const bf16*)w_gate,
              (const bf16*)w_up, w_expert_stride, perm, top, plan, E, act, ff, H, limit, alpha, offset,
              mma_vec_ok(x, x_stride, w_gate, w_up, H));
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_moe_down(const void* act, const void* w_down, long long w_expert_stride, const int* plan, int E,
                           float* y, int n_entries, int H, int ff, int tile_rows, int dtype, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (tile_rows == FEW_ROWS) {
    if (dtype != MI_DTYPE_BF16 || !mma_vec_ok(act, ff, w_down, nullptr, ff))
      MI_REFUSE("moe: the streaming product takes bfloat16 rows of whole 16-byte pieces");
    dim3 g((H + 7) / 8, max_tiles(n_entries, E, FEW_ROWS));
    if (g.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
    MI_LAUNCH((moe_stream_kernel<false>), g, 256, 0, stream, (const bf16*)act, ff, (const bf16*)w_down,
              (const bf16*)nullptr, w_expert_stride, (const int*)nullptr, 1, plan, E, (void*)y, H, ff, 0.f, 0.f, 0.f);
    MI_RETURN_LAUNCH_STATUS();
  }
  dim3 grid((H + TILE_N - 1) / TILE_N, max_tiles(n_entries, E, TILE_M));
  if (grid.y > 65535) MI_REFUSE("moe: too many row tiles for one launch");
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_gemm_kernel<float, false>), grid, 256, 0, stream, (const float*)act, ff, (const float*)w_down,
              (const float*)nullptr, w_expert_stride, (const int*)nullptr, 1, plan, E, (void*)y, H, ff, 0.f, 0.f, 0.f);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_gemm_mma_kernel<false>), grid, 128, 0, stream, (const bf16*)act, ff, (const bf16*)w_down,
              (const bf16*)nullptr, w_expert_stride, (const int*)nullptr, 1, plan, E, (void*)y, H, ff, 0.f, 0.f, 0.f,
              mma_vec_ok(act, ff, w_down, nullptr, ff));
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ gather, combine
// xs[pos, :] = x[perm[pos] / top, :]: an expert's rows side by side, for a library's grouped product
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ perm, int top,
                                  T* __restrict__ xs, int H, int vec) {
  mi_pdl_enter();
  const int pos = blockIdx.x;
  const T* src = x + (size_t)(perm[pos] / top) * x_stride;
  T* dst = xs + (size_t)pos * H;
  if (vec) {
    constexpr int EPC = 16 / (int)sizeof(T);
    for (int c = threadIdx.x * EPC; c < H; c += blockDim.x * EPC)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
  }
}

extern "C" int mi_moe_gather(const void* x, int x_stride, const int* perm, int top, void* xs, int n, int H, int dtype,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  const int es = dtype == MI_DTYPE_F32 ? 4 : 2;
  const int epc = 16 / es;
  const int vec = (H % epc == 0) && (x_stride % epc == 0) && mi_aligned(x, 16) && mi_aligned(xs, 16);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_gather_kernel<float>), n, 128, 0, stream, (const float*)x, x_stride, perm, top, (float*)xs, H, vec);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_gather_kernel<bf16>), n, 128, 0, stream, (const bf16*)x, x_stride, perm, top, (bf16*)xs, H, vec);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

template <typename T, typename YT>
__global__ void moe_combine_kernel(const YT* __restrict__ y, const int* __restrict__ inv,
                                   const float* __restrict__ weights, const T* __restrict__ shared, int shared_stride,
                                   T* __restrict__ out, int H, int top, const float* __restrict__ shared_gate,
                                   int gate_stride) {
  mi_pdl_enter();
  const int t = blockIdx.x;
  // shared_gate: one fp32 number per token whose sigmoid multiplies the shared expert's output
  const float sg = (shared && shared_gate) ? 1.f / (1.f + expf(-shared_gate[(size_t)t * gate_stride])) : 1.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(size_t)t * top + k], mi_to_float(y[(size_t)inv[(size_t)t * top + k] * H + c]), acc);
    if (shared) acc = fmaf(sg, mi_to_float(shared[(size_t)t * shared_stride + c]), acc);
    out[(size_t)t * H + c] = mi_from_float<T>(acc);
  }
}

// y_dtype: the experts' outputs are fp32 (own products) or in the compute dtype (a library's grouped product)
extern "C" int mi_moe_combine(const void* y, int y_dtype, const int* inv, const float* weights, const void* shared,
                              int shared_stride, void* out, int M, int H, int top, const float* shared_gate,
                              int gate_stride, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == MI_DTYPE_F32 && y_dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_combine_kernel<float, float>), M, threads, 0, stream, (const float*)y, inv, weights,
              (const float*)shared, shared_stride, (float*)out, H, top, shared_gate, gate_stride);
  else if (dtype == MI_DTYPE_BF16 && y_dtype == MI_DTYPE_F32)
    MI_LAUNCH((moe_combine_kernel<bf16, float>), M, threads, 0, stream, (const float*)y, inv, weights,
              (const bf16*)shared, shared_stride, (bf16*)out, H, top, shared_gate, gate_stride);
  else if (dtype == MI_DTYPE_BF16 && y_dtype == MI_DTYPE_BF16)
    MI_LAUNCH((moe_combine_kernel<bf16, bf16>), M, threads, 0, stream, (const bf16*)y, inv, weights,
              (const bf16*)shared, shared_stride, (bf16*)out, H, top, shared_gate, gate_stride);
  else
    MI_REFUSE("moe: unsupported dtypes %d (activations) and %d (expert outputs)", dtype, y_dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------------------ dense expert
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, int stride, T* __restrict__ out, int M, int I,
                                   float limit, float alpha, float offset) {
  mi_pdl_enter();
  const size_t n = (size_t)M * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / I), c = (int)(idx - (size_t)t * I);
    const float g = mi_to_float(gu[(size_t)t * stride + c]), u = mi_to_float(gu[(size_t)t * stride + I + c]);
    out[idx] = mi_from_float<T>(mi_clamped_glu_value(g, u, limit, alpha, offset));
  }
}

extern "C" int mi_clamped_glu(const void* gu, int stride, void* out, int M, int I, float limit, float alpha,
                              float offset, int dtype, cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  const size_t n = (size_t)M * I;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((clamped_glu_kernel<float>), blocks, 256, 0, stream, (const float*)gu, stride, (float*)out, M, I, limit, alpha, offset);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((clamped_glu_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gu, stride, (bf16*)out, M, I, limit, alpha, offset);
  else
    MI_REFUSE("moe: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}
