// Routed feed-forward (mixture of experts) without a host round trip:
//
//   moe_route     per token: scores from the 32-bit router logits (sigmoid, or softmax over the experts), the
//                 `top` largest (ties: the lower index), their weights (the scores, optionally renormalized);
//                 with a `correction` per expert the CHOICE goes by score + correction, the weight stays the score
//   moe_arrange   the (token, choice) pairs grouped by expert: offsets[E + 1], sorted[p] = pair at place p,
//                 place[pair] = p
//   moe_grouped_linear   for every expert e and every place p of it:  out[p] = f(W_e . (s_p * x[row(p)]))
//                 with W_e = weights[e]; GATED: W_e stacks gate rows on up rows and
//                 out[p] = act(s_p * gate . x) * (s_p * up . x); s_p = the pair's weight when the weight
//                 multiplies the expert's input, else 1
//   moe_combine   y[t] = sum over the token's choices (in choice order) of c * rows[place], c = the weight when it
//                 multiplies the expert's output, else 1.  A choice at or beyond `experts` (an expert without
//                 tensors that passes its input) adds c * x[t]; a shared expert's rows, if given, are added times
//                 sigmoid of one 32-bit number per token
//
// Gate activations of the grouped product: 0 silu(g) u, 1 gelu_tanh(g) u, 2 the clamped form
// g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit).
//
// The grouped product is a tiled kernel with 32-bit accumulation for float32 and 16-bit storage alike; a block
// finds its (expert, row tile) from the offsets, so the grid depends only on the step's size.
#include "common.cuh"

#define MOE_MAX_TOP 32

__global__ void moe_route_kernel(const float* __restrict__ logits, long long logits_stride,
                                 const float* __restrict__ correction, int* __restrict__ choice,
                                 float* __restrict__ weight, int tokens, int experts, int top, int softmax_scores,
                                 int renormalize) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* z = logits + (long long)t * logits_stride;
  float zmax = -INFINITY, zsum = 0.f;
  if (softmax_scores) {
    for (int e = lane; e < experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    for (int e = lane; e < experts; e += 32) zsum += expf(z[e] - zmax);
    zsum = warp_sum(zsum);
  }
  int taken[MOE_MAX_TOP];
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.f;  // the choice's rank (score + correction) and its score
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      bool used = false;
      for (int j = 0; j < k; ++j) used |= taken[j] == e;
      if (used) continue;
      const float s = softmax_scores ? expf(z[e] - zmax) / zsum : 1.f / (1.f + expf(-z[e]));
      const float rank = correction != nullptr ? s + correction[e] : s;
      if (rank > best || (rank == best && e < best_e)) {
        best = rank;
        best_s = s;
        best_e = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_s = os;
        best_e = oe;
      }
    }
    taken[k] = best_e;
    total += best_s;
    if (lane == 0) {
      choice[(long long)t * top + k] = best_e;
      weight[(long long)t * top + k] = best_s;
    }
  }
  if (renormalize && lane == 0)
    for (int k = 0; k < top; ++k) weight[(long long)t * top + k] /= total;
}

// One block.  counts in shared memory (experts <= 1024).
__global__ void moe_arrange_kernel(const int* __restrict__ choice, int pairs, int experts, int* __restrict__ offsets,
                                   int* __restrict__ sorted, int* __restrict__ place) {
  __shared__ int count[1024];
  __shared__ int cursor[1024];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = choice[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += count[e];
    }
    offsets[experts] = run;
  }
  __syncthreads();
  // the order inside an expert's group has no influence on any result: every place is computed by itself
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = choice[p];
    if (e >= 0 && e < experts) {
      const int at = atomicAdd(&cursor[e], 1);
      sorted[at] = p;
      place[p] = at;
    }
  }
}

__device__ __forceinline__ float moe_gate_act(int act, float g, float u, float limit, float alpha) {
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
  }
  return (act == 0 ? act_silu(g) : act_gelu_tanh(g)) * u;
}

#define MOE_BM 32
#define MOE_BN 64
#define MOE_BK 32
#define MOE_THREADS 256  // a thread: 2 rows x 4 columns of the tile

template <typename T, bool GATED>
__global__ void __launch_bounds__(MOE_THREADS)
moe_grouped_linear_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ weights,
                          long long expert_stride, const int* __restrict__ offsets, const int* __restrict__ sorted,
                          const float* __restrict__ pair_weight, T* __restrict__ out, int experts, int top,
                          int rows_from_pairs, int n_out, int k_dim, int act, float limit, float alpha) {
  __shared__ float As[MOE_BK][MOE_BM + 1];
  __shared__ float Bs[GATED ? 2 : 1][MOE_BK][MOE_BN + 1];
  __shared__ int s_row[MOE_BM];
  __shared__ float s_scale[MOE_BM];
  pdl_launch_dependents();
  pdl_wait();
  // which expert and which tile of its rows
  int e = 0, tile = blockIdx.y, lo = 0, hi = 0;
  for (; e < experts; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int tiles = (hi - lo + MOE_BM - 1) / MOE_BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= experts) return;
  const int p0 = lo + tile * MOE_BM;
  const int rows = min(MOE_BM, hi - p0);
  const int n0 = blockIdx.x * MOE_BN;
  if (threadIdx.x < MOE_BM) {
    const int i = threadIdx.x;
    int src = 0;
    float sc = 0.f;
    if (i < rows) {
      const int pair = sorted[p0 + i];
      src = rows_from_pairs ? pair / top : p0 + i;  // the token's row of x, or the place's own row
      sc = pair_weight != nullptr ? pair_weight[pair] : 1.f;
    }
    s_row[i] = src;
    s_scale[i] = sc;
  }
  __syncthreads();
  const T* W = weights + (long long)e * expert_stride;
  const int tr = threadIdx.x / 16, tc = threadIdx.x % 16;  // rows tr*2.., columns tc*4..
  float acc[GATED ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  for (int k0 = 0; k0 < k_dim; k0 += MOE_BK) {
    for (int idx = threadIdx.x; idx < MOE_BM * MOE_BK; idx += MOE_THREADS) {
      const int i = idx / MOE_BK, kk = idx % MOE_BK;
      float v = 0.f;
      if (i < rows && k0 + kk < k_dim) v = to_f32(x[(long long)s_row[i] * x_stride + k0 + kk]);
      As[kk][i] = v;
    }
    for (int idx = threadIdx.x; idx < MOE_BN * MOE_BK; idx += MOE_THREADS) {
      const int j = idx / MOE_BK, kk = idx % MOE_BK;
      const bool on = n0 + j < n_out && k0 + kk < k_dim;
      Bs[0][kk][j] = on ? to_f32(W[(long long)(n0 + j) * k_dim + k0 + kk]) : 0.f;
      if (GATED) Bs[1][kk][j] = on ? to_f32(W[(long long)(n_out + n0 + j) * k_dim + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MOE_BK; ++kk) {
      const float a0 = As[kk][tr * 2], a1 = As[kk][tr * 2 + 1];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = Bs[g][kk][tc * 4 + j];
          acc[g][0][j] = fmaf(a0, b, acc[g][0][j]);
          acc[g][1][j] = fmaf(a1, b, acc[g][1][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = tr * 2 + i;
    if (r >= rows) continue;
    const float sc = s_scale[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tc * 4 + j;
      if (c >= n_out) continue;
      float v;
      if (GATED) {
        const float g = acc[0][i][j] * sc, u = acc[1][i][j] * sc;
        v = moe_gate_act(act, g, u, limit, alpha);
      } else {
        v = acc[0][i][j] * sc;
      }
      out[(long long)(p0 + r) * n_out + c] = from_f32<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------
// The grouped product on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit accumulation): a block owns 64
// places of one expert x 64 output columns (gate and up columns both when GATED); x rows (gathered by place) and
// weight rows go through a two-stage cp.async ring of 64-element k slices in 128-byte rows with the chunk index
// XORed by the row (conflict-free ldmatrix).  Needs k_dim, the row stride of x and n_out to allow 16-byte pieces
// and paired stores; the launcher falls back to the kernel above otherwise.
// ---------------------------------------------------------------------------
#define MMA_BM 64
#define MMA_BN 64
#define MMA_BK 64
#define MMA_THREADS 128

__device__ __forceinline__ void moe_cp_async_16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void moe_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void moe_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void moe_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void moe_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED, int STAGES>
__global__ void __launch_bounds__(MMA_THREADS)
moe_grouped_mma_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                       const __nv_bfloat16* __restrict__ weights, long long expert_stride,
                       const int* __restrict__ offsets, const int* __restrict__ sorted,
                       const float* __restrict__ pair_weight, __nv_bfloat16* __restrict__ out, int experts, int top,
                       int rows_from_pairs, int n_out, int k_dim, int act, float limit, float alpha) {
  constexpr int NB = GATED ? 2 : 1;
  constexpr int TILE = MMA_BM * MMA_BK * 2;  // bytes of one 64 x 64 tile
  extern __shared__ __align__(128) unsigned char moe_smem[];
  __shared__ int s_row[MMA_BM];
  __shared__ float s_scale[MMA_BM];
  pdl_launch_dependents();
  pdl_wait();
  int e = 0, tile = blockIdx.y, lo = 0, hi = 0;
  for (; e < experts; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int tiles = (hi - lo + MMA_BM - 1) / MMA_BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e >= experts) return;
  const int p0 = lo + tile * MMA_BM;
  const int rows = min(MMA_BM, hi - p0);
  const int n0 = blockIdx.x * MMA_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MMA_BM) {
    int src = 0;
    float sc = 0.f;
    if (tid < rows) {
      const int pair = sorted[p0 + tid];
      src = rows_from_pairs ? pair / top : p0 + tid;
      sc = pair_weight != nullptr ? pair_weight[pair] : 1.f;
    }
    s_row[tid] = src;
    s_scale[tid] = sc;
  }
  __syncthreads();
  const __nv_bfloat16* W = weights + (long long)e * expert_stride;
  unsigned char* a_s = moe_smem;                      // [STAGES][TILE]
  unsigned char* b_s = moe_smem + STAGES * TILE;      // [STAGES][NB][TILE]
  const int ksteps = (k_dim + MMA_BK - 1) / MMA_BK;

  auto issue = [&](int kt) {
    const int st = kt % STAGES;
    const int k0 = kt * MMA_BK;
#pragma unroll
    for (int i = 0; i < MMA_BM * 8 / MMA_THREADS; ++i) {
      const int c = i * MMA_THREADS + tid;
      const int row = c >> 3, ch = c & 7;
      const bool k_ok = k0 + ch * 8 < k_dim;
      const int sw = row * 128 + ((ch ^ (row & 7)) * 16);
      const bool a_ok = k_ok && row < rows;
      moe_cp_async_16(a_s + st * TILE + sw, x + (a_ok ? (long long)s_row[row] * x_stride + k0 + ch * 8 : 0), a_ok);
      const bool b_ok = k_ok && n0 + row < n_out;
#pragma unroll
      for (int g = 0; g < NB; ++g)
        moe_cp_async_16(b_s + (st * NB + g) * TILE + sw,
                        W + (b_ok ? ((long long)(g * n_out + n0 + row) * k_dim + k0 + ch * 8) : 0), b_ok);
    }
  };

  float acc[NB][8][4];
#pragma unroll
  for (int g = 0; g < NB; ++g)
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[g][t][0] = acc[g][t][1] = acc[g][t][2] = acc[g][t][3] = 0.f;

  // a ring of STAGES k slices: STAGES - 1 are in flight while one is multiplied (2 for steps of many rows, where
  // the blocks of an SM hide one another's loads; 4 for steps of few rows, where a block streams its weights alone)
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < ksteps) issue(i);
    moe_commit();
  }
  for (int kt = 0; kt < ksteps; ++kt) {
    if (kt + STAGES - 1 < ksteps) issue(kt + STAGES - 1);
    moe_commit();
    moe_wait<STAGES - 1>();
    __syncthreads();
    const unsigned char* at = a_s + (kt % STAGES) * TILE;
#pragma unroll
    for (int kk = 0; kk < MMA_BK / 16; ++kk) {
      unsigned a[4];
      {
        const int mat = lane >> 3, row = warp * 16 + (mat & 1) * 8 + (lane & 7), ch = 2 * kk + (mat >> 1);
        moe_ldsm4(a[0], a[1], a[2], a[3], at + row * 128 + ((ch ^ (row & 7)) * 16));
      }
#pragma unroll
      for (int g = 0; g < NB; ++g) {
        const unsigned char* bt = b_s + ((kt % STAGES) * NB + g) * TILE;
#pragma unroll
        for (int t = 0; t < 8; t += 2) {
          const int mat = lane >> 3, row = t * 8 + (mat >> 1) * 8 + (lane & 7), ch = 2 * kk + (mat & 1);
          unsigned b0, b1, b2, b3;
          moe_ldsm4(b0, b1, b2, b3, bt + row * 128 + ((ch ^ (row & 7)) * 16));
          moe_mma(acc[g][t], a, b0, b1);
          moe_mma(acc[g][t + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    if (r >= rows) continue;
    const float sc = s_scale[r];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int c = n0 + t * 8 + (lane & 3) * 2;
      if (c >= n_out) continue;  // (n_out is even: a pair is inside or outside)
      float v[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (GATED) {
          const float gt = acc[0][t][2 * h + j] * sc, up = acc[NB - 1][t][2 * h + j] * sc;
          v[j] = moe_gate_act(act, gt, up, limit, alpha);
        } else {
          v[j] = acc[0][t][2 * h + j] * sc;
        }
      }
      *reinterpret_cast<__nv_bfloat162*>(out + (long long)(p0 + r) * n_out + c) = __floats2bfloat162_rn(v[0], v[1]);
    }
  }
}

// VEC elements of T from p to 32-bit: one 16-byte load when VEC elements are 16 bytes, else element by element.
template <typename T, int VEC>
__device__ __forceinline__ void moe_load_vec(const T* __restrict__ p, float (&out)[VEC]) {
  if constexpr (VEC * sizeof(T) == 16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = to_f32(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = to_f32(p[i]);
  }
}

// A block: one token x (blockDim.x * VEC) columns (blockIdx.y counts the column ranges); a thread: VEC columns.
template <typename T, int VEC>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place,
                                   const float* __restrict__ pair_weight, T* __restrict__ y, int top, int cols,
                                   const int* __restrict__ choice, int experts, const T* __restrict__ x,
                                   long long x_stride, const T* __restrict__ shared_rows,
                                   const float* __restrict__ shared_gate, long long gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= cols) return;
  float acc[VEC], v[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  for (int k = 0; k < top; ++k) {
    const long long pair = t * top + k;
    const bool passes = choice != nullptr && choice[pair] >= experts;  // an expert that is its input
    const T* src = passes ? x + t * x_stride : rows + (long long)place[pair] * cols;
    moe_load_vec<T, VEC>(src + c0, v);
    const float w = pair_weight != nullptr ? pair_weight[pair] : 1.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] += w * v[i];
  }
  if (shared_rows != nullptr) {
    const float sg = shared_gate != nullptr ? 1.f / (1.f + expf(-shared_gate[t * gate_stride])) : 1.f;
    moe_load_vec<T, VEC>(shared_rows + t * cols + c0, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] += sg * v[i];
  }
  if constexpr (VEC * sizeof(T) == 16) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = from_f32<T>(acc[i]);
    *reinterpret_cast<uint4*>(y + t * cols + c0) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) y[t * cols + c0 + i] = from_f32<T>(acc[i]);
  }
}

// The same sum, added to a 32-bit residual stream instead of stored, with a scale per channel, and followed by the
// RMS norm that reads the stream next:  stream[t] += scale * y[t];  out[t] = w2 * stream[t] / sqrt(mean(stream[t]^2) +
// eps2).  One block per token; the sum never leaves 32-bit.  `x` (the passing experts' input) and `out` may be the
// same rows: a block reads its token's row of x before the barrier and writes its row of out behind it.
template <typename T, int VEC>
__global__ void moe_combine_add_norm_kernel(const T* __restrict__ rows, const int* __restrict__ place,
                                            const float* __restrict__ pair_weight, int top, int cols,
                                            const int* __restrict__ choice, int experts, const T* x,
                                            long long x_stride, const T* __restrict__ shared_rows,
                                            const float* __restrict__ shared_gate, long long gate_stride,
                                            float* __restrict__ stream, const float* __restrict__ scale,
                                            const float* __restrict__ w2, float eps2, T* out) {
  extern __shared__ __align__(16) float mc_row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const float sg = (shared_rows != nullptr && shared_gate != nullptr)
                       ? 1.f / (1.f + expf(-shared_gate[t * gate_stride])) : 1.f;
  float sq = 0.f;
  for (int c0 = threadIdx.x * VEC; c0 < cols; c0 += blockDim.x * VEC) {
    float acc[VEC], v[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int k = 0; k < top; ++k) {
      const long long pair = t * top + k;
      const bool passes = choice != nullptr && choice[pair] >= experts;
      const T* src = passes ? x + t * x_stride : rows + (long long)place[pair] * cols;
      moe_load_vec<T, VEC>(src + c0, v);
      const float w = pair_weight != nullptr ? pair_weight[pair] : 1.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += w * v[i];
    }
    if (shared_rows != nullptr) {
      moe_load_vec<T, VEC>(shared_rows + t * cols + c0, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += sg * v[i];
    }
    if constexpr (VEC % 4 == 0) {
      // (c0 is a multiple of VEC, cols too: 16-byte pieces of the stream, the scale and the row in shared memory)
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        float4 s4 = *reinterpret_cast<const float4*>(stream + t * cols + c0 + i);
        float4 sc = make_float4(1.f, 1.f, 1.f, 1.f);
        if (scale != nullptr) sc = *reinterpret_cast<const float4*>(scale + c0 + i);
        s4.x += sc.x * acc[i];
        s4.y += sc.y * acc[i + 1];
        s4.z += sc.z * acc[i + 2];
        s4.w += sc.w * acc[i + 3];
        *reinterpret_cast<float4*>(stream + t * cols + c0 + i) = s4;
        *reinterpret_cast<float4*>(mc_row + c0 + i) = s4;
        sq += s4.x * s4.x + s4.y * s4.y + s4.z * s4.z + s4.w * s4.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int c = c0 + i;
        const float s = stream[t * cols + c] + (scale != nullptr ? scale[c] : 1.f) * acc[i];
        stream[t * cols + c] = s;
        mc_row[c] = s;
        sq += s * s;
      }
    }
  }
  if (out == nullptr) return;
  const float rstd = 1.f / sqrtf(block_sum(sq, scratch) / (float)cols + eps2);
  if constexpr (VEC * sizeof(T) == 16) {
    for (int c0 = threadIdx.x * VEC; c0 < cols; c0 += blockDim.x * VEC) {
      uint4 raw;
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) e[i] = from_f32<T>(mc_row[c0 + i] * rstd * w2[c0 + i]);
      *reinterpret_cast<uint4*>(out + t * cols + c0) = raw;
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[t * cols + c] = from_f32<T>(mc_row[c] * rstd * w2[c]);
  }
}

static int g_moe_force_plain = 0;
// 1: the grouped product never takes the tensor-core kernel (tests compare the two)
extern "C" void ullm_moe_force_plain(int on) { g_moe_force_plain = on ? 1 : 0; }

// `logits_stride`: floats between two tokens' rows (the rows may hold further columns behind the experts');
// `correction` (null: none): added to the scores for the choice only.
extern "C" int ullm_moe_route(const float* logits, long long logits_stride, const float* correction, int* choice,
                              float* weight, int tokens, int experts, int top, int softmax_scores, int renormalize,
                              void* stream) {
  if (tokens < 0 || experts <= 0 || top <= 0 || logits_stride < experts) return ULLM_ERR_BAD_SIZE;
  if (top > experts || top > MOE_MAX_TOP) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  return ullm_launch_kernel(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, (cudaStream_t)stream, logits,
                            logits_stride, correction, choice, weight, tokens, experts, top, softmax_scores,
                            renormalize);
}

extern "C" int ullm_moe_arrange(const int* choice, int pairs, int experts, int* offsets, int* sorted, int* place,
                                void* stream) {
  if (pairs < 0 || experts <= 0) return ULLM_ERR_BAD_SIZE;
  if (experts > 1024) return ULLM_ERR_UNSUPPORTED;
  return ullm_launch_kernel(moe_arrange_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, choice, pairs, experts,
                            offsets, sorted, place);
}

template <typename T>
static int grouped_launch(const void* x, long long x_stride, const void* weights, long long expert_stride,
                          const int* offsets, const int* sorted, const float* pair_weight, void* out, int pairs,
                          int experts, int top, int rows_from_pairs, int n_out, int k_dim, int gated, int act,
                          float limit, float alpha, cudaStream_t st) {
  const int row_tiles = (pairs + MOE_BM - 1) / MOE_BM + experts;  // an upper bound whatever the routing
  const dim3 grid((n_out + MOE_BN - 1) / MOE_BN, row_tiles), block(MOE_THREADS);
  if (gated)
    return ullm_launch_kernel(moe_grouped_linear_kernel<T, true>, grid, block, 0, st, (const T*)x, x_stride,
                              (const T*)weights, expert_stride, offsets, sorted, pair_weight, (T*)out, experts, top,
                              rows_from_pairs, n_out, k_dim, act, limit, alpha);
  return ullm_launch_kernel(moe_grouped_linear_kernel<T, false>, grid, block, 0, st, (const T*)x, x_stride,
                            (const T*)weights, expert_stride, offsets, sorted, pair_weight, (T*)out, experts, top,
                            rows_from_pairs, n_out, k_dim, act, limit, alpha);
}

// x: rows of k_dim elements (stride x_stride); row of place p = token of its pair (rows_from_pairs) or p itself.
// weights: [experts, (gated ? 2 : 1) * n_out, k_dim].  out: [pairs, n_out].
extern "C" int ullm_moe_grouped_linear(int dtype, const void* x, long long x_stride, const void* weights,
                                       long long expert_stride, const int* offsets, const int* sorted,
                                       const float* pair_weight, void* out, int pairs, int experts, int top,
                                       int rows_from_pairs, int n_out, int k_dim, int gated, int act, float limit,
                                       float alpha, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (pairs < 0 || experts <= 0 || top <= 0 || n_out <= 0 || k_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (gated && (act < 0 || act > 2)) return ULLM_ERR_UNSUPPORTED;
  if (gated && act == 2 && !(limit > 0.f)) return ULLM_ERR_BAD_SIZE;
  if (pairs == 0) return ULLM_OK;
  if ((pairs + MOE_BM - 1) / MOE_BM + experts > 65535) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32)
    return grouped_launch<float>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out, pairs,
                                 experts, top, rows_from_pairs, n_out, k_dim, gated, act, limit, alpha, st);
  if (dtype == ULLM_DTYPE_BF16) {
    const bool tensor_cores = !g_moe_force_plain && k_dim % 8 == 0 && x_stride % 8 == 0 && n_out % 2 == 0 &&
                              (uintptr_t)x % 16 == 0 && (uintptr_t)weights % 16 == 0 && (uintptr_t)out % 4 == 0 &&
                              expert_stride % 8 == 0;
    if (tensor_cores) {
      const int row_tiles = (pairs + MMA_BM - 1) / MMA_BM + experts;
      if (row_tiles > 65535) return ULLM_ERR_BAD_SIZE;
      const dim3 grid((n_out + MMA_BN - 1) / MMA_BN, row_tiles), block(MMA_THREADS);
      // steps of few rows: every block streams its expert's weights nearly alone, so more of them are kept in flight
      const int stages = pairs <= 256 ? 4 : 2;
      const size_t smem = (size_t)stages * (1 + (gated ? 2 : 1)) * MMA_BM * MMA_BK * 2;
      static int attr_set = 0;
      if (!attr_set) {  // (with the static arrays the gated form is just above the size a kernel gets unasked)
        if (cudaFuncSetAttribute(moe_grouped_mma_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(moe_grouped_mma_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(moe_grouped_mma_kernel<true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(moe_grouped_mma_kernel<false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess)
          return ULLM_ERR_LAUNCH;
        attr_set = 1;
      }
#define MMA_GO(G, S)                                                                                                  \
  return ullm_launch_kernel(moe_grouped_mma_kernel<G, S>, grid, block, smem, st, (const __nv_bfloat16*)x, x_stride,    \
                            (const __nv_bfloat16*)weights, expert_stride, offsets, sorted, pair_weight,               \
                            (__nv_bfloat16*)out, experts, top, rows_from_pairs, n_out, k_dim, act, limit, alpha)
      if (gated && stages == 4) MMA_GO(true, 4);
      if (gated) MMA_GO(true, 2);
      if (stages == 4) MMA_GO(false, 4);
      MMA_GO(false, 2);
#undef MMA_GO
    }
    return grouped_launch<__nv_bfloat16>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out,
                                         pairs, experts, top, rows_from_pairs, n_out, k_dim, gated, act, limit, alpha, st);
  }
  if (dtype == ULLM_DTYPE_F16)
    return grouped_launch<__half>(x, x_stride, weights, expert_stride, offsets, sorted, pair_weight, out, pairs,
                                  experts, top, rows_from_pairs, n_out, k_dim, gated, act, limit, alpha, st);
  return ULLM_ERR_BAD_DTYPE;
}

// `choice` with `experts` and `x` (null: every choice has rows): a choice >= experts adds the weight times the
// token's row of x.  `shared_rows` (null: none): added times sigmoid(shared_gate[t * gate_stride]) (gate null: 1).
extern "C" int ullm_moe_combine(int dtype, const void* rows, const int* place, const float* pair_weight, void* y,
                                int tokens, int top, int cols, const int* choice, int experts, const void* x,
                                long long x_stride, const void* shared_rows, const float* shared_gate,
                                long long gate_stride, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || top <= 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if (choice != nullptr && (x == nullptr || x_stride < cols || experts < 0)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const int esize = dtype == ULLM_DTYPE_F32 ? 4 : 2;
  const int vec = 16 / esize;
  const bool wide = cols % vec == 0 && x_stride % vec == 0 &&
                    (((uintptr_t)rows | (uintptr_t)y | (uintptr_t)x | (uintptr_t)shared_rows) & 15) == 0;
  const int per_thread = wide ? vec : 1;
  int threads = 32;
  while (threads < 128 && threads * per_thread < cols) threads <<= 1;
  const dim3 grid(tokens, (cols + threads * per_thread - 1) / (threads * per_thread)), block(threads);
#define MC_GO(T, V)                                                                                                 \
  return ullm_launch_kernel(moe_combine_kernel<T, V>, grid, block, 0, st, (const T*)rows, place, pair_weight, (T*)y, \
                            top, cols, choice, experts, (const T*)x, x_stride, (const T*)shared_rows, shared_gate,  \
                            gate_stride)
  if (dtype == ULLM_DTYPE_F32) {
    if (wide) MC_GO(float, 4);
    MC_GO(float, 1);
  }
  if (dtype == ULLM_DTYPE_BF16) {
    if (wide) MC_GO(__nv_bfloat16, 8);
    MC_GO(__nv_bfloat16, 1);
  }
  if (dtype == ULLM_DTYPE_F16) {
    if (wide) MC_GO(__half, 8);
    MC_GO(__half, 1);
  }
#undef MC_GO
  return ULLM_ERR_BAD_DTYPE;
}

// stream (32-bit, [tokens, cols], in place) += scale * (the sum `ullm_moe_combine` forms); `scale` null: 1.  `out` with
// `w2` (null: none): the RMS norm of the updated rows, in the rows' dtype; `out` may be `x`.
extern "C" int ullm_moe_combine_add_norm(int dtype, const void* rows, const int* place, const float* pair_weight,
                                         int tokens, int top, int cols, const int* choice, int experts, const void* x,
                                         long long x_stride, const void* shared_rows, const float* shared_gate,
                                         long long gate_stride, float* stream_rows, const float* scale,
                                         const float* w2, float eps2, void* out, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || top <= 0 || cols <= 0 || stream_rows == nullptr) return ULLM_ERR_BAD_SIZE;
  if (choice != nullptr && (x == nullptr || x_stride < cols || experts < 0)) return ULLM_ERR_BAD_SIZE;
  if (out != nullptr && w2 == nullptr) return ULLM_ERR_BAD_SIZE;
  const size_t smem = (size_t)cols * sizeof(float);
  if (smem > 160 * 1024) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const int esize = dtype == ULLM_DTYPE_F32 ? 4 : 2;
  const int vec = 16 / esize;
  const bool wide = cols % vec == 0 && x_stride % vec == 0 &&
                    (((uintptr_t)rows | (uintptr_t)x | (uintptr_t)shared_rows | (uintptr_t)stream_rows |
                      (uintptr_t)scale | (uintptr_t)w2 | (uintptr_t)out) & 15) == 0;
  const int per_thread = wide ? vec : 1;
  int threads = 32;
  while (threads < 256 && threads * per_thread < cols) threads <<= 1;
  const dim3 grid(tokens), block(threads);
#define MCA_GO(T, V)                                                                                                   \
  {                                                                                                                    \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(moe_combine_add_norm_kernel<T, V>,                                    \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
      cudaGetLastError();                                                                                              \
      return ULLM_ERR_LAUNCH;                                                                                          \
    }                                                                                                                  \
    return ullm_launch_kernel(moe_combine_add_norm_kernel<T, V>, grid, block, smem, st, (const T*)rows, place,         \
                              pair_weight, top, cols, choice, experts, (const T*)x, x_stride, (const T*)shared_rows,   \
                              shared_gate, gate_stride, stream_rows, scale, w2, eps2, (T*)out);                        \
  }
  if (dtype == ULLM_DTYPE_F32) {
    if (wide) MCA_GO(float, 4);
    MCA_GO(float, 1);
  }
  if (dtype == ULLM_DTYPE_BF16) {
    if (wide) MCA_GO(__nv_bfloat16, 8);
    MCA_GO(__nv_bfloat16, 1);
  }
  if (dtype == ULLM_DTYPE_F16) {
    if (wide) MCA_GO(__half, 8);
    MCA_GO(__half, 1);
  }
#undef MCA_GO
  return ULLM_ERR_BAD_DTYPE;
}
