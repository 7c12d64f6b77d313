// Preparation kernels of three attention forms, each in front of the general attention kernel:
//
//   kv_shared_prepare   attention whose VALUES ARE ITS KEYS as projected (no value projection), with an optional
//                       RMS norm of q and of k over the WHOLE projection (all heads at once, one weight per
//                       channel): q is normed in place, the normed k goes to the key pages and the k as projected
//                       to the value pages; without the norm only the key pages are written (the values are read
//                       from them)
//   pool_blocks         mean key / value of each block of P positions whose last position arrived in this step,
//                       read from the pages as they hold them, written to pooled pages of their own
//   latent_prepare      latent attention in its absorbed form: the latent c = RMSnorm(first `rank` columns of the
//                       down projection) and the rotated shared key part form ONE key row [c | k_rot] of a single
//                       kv head (the values are its first `rank` elements); a query row per head is
//                       [q_h W_uk,h (from a batched product) | rotated q_rot,h]
//
//   qkv_rows_prepare    grouped attention with q | k | v projections: an optional RMS norm of q and of k over the
//                       WHOLE projection (a weight per channel), then the rotation of the first `rot_dims`
//                       dimensions of every q and k head, a factor per query head on q, and every value head
//                       divided by its root mean square (no weight); q goes to a buffer of its own, k and v to
//                       their pages
//
// Rotation: with `interleaved` neighbours (2i, 2i + 1), otherwise (i, i + dims / 2), i < dims / 2, turn by the
// 32-bit angle position * f_i (f_i from a table built in 64-bit); sincosf is the accurate form.  Sums and norms
// are 32-bit; one rounding at each store.
#include "common.cuh"

// One block per token.  qk: [tokens][stride], q in columns 0 .. q_size-1, k in q_size .. q_size + kv_size - 1.
template <typename T>
__global__ void kv_shared_prepare_kernel(T* __restrict__ qk, long long stride, int q_size, int kv_size,
                                         const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                         const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages, long long num_slots, int* status) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  T* q = qk + (long long)t * stride;
  T* k = q + q_size;
  long long slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
    slot = -1;
  }
  if (wq != nullptr) {
    float acc = 0.f;
    for (int c = threadIdx.x; c < q_size; c += blockDim.x) {
      const float v = to_f32(q[c]);
      acc += v * v;
    }
    const float rq = 1.f / sqrtf(block_sum(acc, scratch) / (float)q_size + eps);
    for (int c = threadIdx.x; c < q_size; c += blockDim.x) q[c] = from_f32<T>(to_f32(q[c]) * rq * wq[c]);
    acc = 0.f;
    for (int c = threadIdx.x; c < kv_size; c += blockDim.x) {
      const float v = to_f32(k[c]);
      acc += v * v;
    }
    const float rk = 1.f / sqrtf(block_sum(acc, scratch) / (float)kv_size + eps);
    if (slot >= 0) {
      for (int c = threadIdx.x; c < kv_size; c += blockDim.x) {
        const T raw = k[c];
        k_pages[slot * kv_size + c] = from_f32<T>(to_f32(raw) * rk * wk[c]);
        if (v_pages != nullptr) v_pages[slot * kv_size + c] = raw;
      }
    }
  } else if (slot >= 0) {
    for (int c = threadIdx.x; c < kv_size; c += blockDim.x) {
      const T raw = k[c];
      k_pages[slot * kv_size + c] = raw;
      if (v_pages != nullptr) v_pages[slot * kv_size + c] = raw;
    }
  }
}

#define POOL_SLOTS 1024
#define ROWS_MAX_ROT 512  // rotated dimensions whose angles a block keeps in shared memory

// One block per token; a token whose pooled slot is -1 completes no block.  The block's positions are
// pos - pool + 1 .. pos of the token's request, found through the request's row of the block table.
template <typename T>
__global__ void pool_blocks_kernel(const int* __restrict__ positions, const int* __restrict__ token_req,
                                   const int* __restrict__ req_slots, const int* __restrict__ block_table,
                                   int max_pages, int page_size, long long num_pages, const T* __restrict__ k_pages,
                                   const T* __restrict__ v_pages, int row, int v_row,
                                   const int* __restrict__ pool_slots, long long num_pool_slots,
                                   T* __restrict__ pk_pages, T* __restrict__ pv_pages, int pool, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const long long dst = pool_slots[t];
  const int r = token_req[t];
  if (dst < 0 || r < 0) return;
  if (dst >= num_pool_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)dst);
    return;
  }
  const int pos = positions[t];
  const int* bt = block_table + (long long)req_slots[r] * max_pages;
  const float inv = 1.f / (float)pool;
  const int cols = row + (v_pages != nullptr ? v_row : 0);
  // blocks of up to POOL_SLOTS positions: their slots are found once; the sums then run over them without a
  // branch, eight loads in flight, in the order of the positions
  __shared__ long long slot_s[POOL_SLOTS];
  if (pool <= POOL_SLOTS) {
    int bad = 0;
    for (int i = threadIdx.x; i < pool; i += blockDim.x) {
      const int j = pos - pool + 1 + i;
      const int page = j >= 0 ? bt[j / page_size] : -1;
      if (page < 0 || page >= num_pages) {
        bad = 1;
        ullm_report(status, ULLM_STATUS_PAGE, t, page);
      } else {
        slot_s[i] = (long long)page * page_size + j % page_size;
      }
    }
    if (__syncthreads_or(bad)) return;  // (nothing is written for a block whose pages are not there)
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const bool is_v = c >= row;
      const T* src = is_v ? v_pages + (c - row) : k_pages + c;
      const long long stride = is_v ? v_row : row;
      float acc = 0.f;
#pragma unroll 8
      for (int i = 0; i < pool; ++i) acc += to_f32(src[slot_s[i] * stride]);
      if (is_v) pv_pages[dst * v_row + (c - row)] = from_f32<T>(acc * inv);
      else pk_pages[dst * row + c] = from_f32<T>(acc * inv);
    }
    return;
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const bool is_v = c >= row;
    float acc = 0.f;
    bool ok = true;
    for (int j = pos - pool + 1; j <= pos; ++j) {
      const int page = j >= 0 ? bt[j / page_size] : -1;
      if (page < 0 || page >= num_pages) {
        ok = false;
        ullm_report(status, ULLM_STATUS_PAGE, t, page);
        break;
      }
      const long long slot = (long long)page * page_size + j % page_size;
      acc += is_v ? to_f32(v_pages[slot * v_row + (c - row)]) : to_f32(k_pages[slot * row + c]);
    }
    if (!ok) continue;
    if (is_v) pv_pages[dst * v_row + (c - row)] = from_f32<T>(acc * inv);
    else pk_pages[dst * row + c] = from_f32<T>(acc * inv);
  }
}

// One block per token.  q_full [tokens][heads][dim + rot] (the query projection; rows `q_stride` apart), q_lat
// [heads][tokens][rank] (q_h W_uk,h; null: already in q_out), dkv [tokens][rank + rot] (rows `dkv_stride` apart);
// q_out [tokens][heads][rank + rot]; key pages [*][rank + rot].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q_full, long long q_stride, const T* __restrict__ q_lat,
                                      const T* __restrict__ dkv, long long dkv_stride, T* __restrict__ q_out,
                                      int tokens, int heads,
                                      int dim, int rot, int rank, int rot_dims, int interleaved,
                                      const float* __restrict__ w_c, float eps, const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                      T* __restrict__ k_pages, long long num_slots, int* status) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float cs_s[ROWS_MAX_ROT / 2], sn_s[ROWS_MAX_ROT / 2];
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  const int kw = rank + rot;
  const int half = rot_dims >> 1;
  // the token's angles once (the launcher refuses more rotated dimensions than the arrays hold)
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &sn_s[i], &cs_s[i]);
  __syncthreads();
  // queries: the absorbed part is copied (unless the product in front wrote it in place), the rotated part turned
  if (q_lat != nullptr) {
    for (int i = threadIdx.x; i < heads * rank; i += blockDim.x) {
      const int h = i / rank, c = i - h * rank;
      q_out[((long long)t * heads + h) * kw + c] = q_lat[((long long)h * tokens + t) * rank + c];
    }
  }
  for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
    const int h = i / rot, c = i - h * rot;
    const T* src = q_full + (long long)t * q_stride + (long long)h * (dim + rot) + dim;
    float v = to_f32(src[c]);
    if (c < rot_dims) {
      const bool second = interleaved ? (c & 1) : (c >= half);
      const int pc = interleaved ? (c ^ 1) : (second ? c - half : c + half);
      const int fi = interleaved ? (c >> 1) : (second ? c - half : c);
      const float sn = sn_s[fi], cs = cs_s[fi];
      const float other = to_f32(src[pc]);
      v = second ? v * cs + other * sn : v * cs - other * sn;
    }
    q_out[((long long)t * heads + h) * kw + rank + c] = from_f32<T>(v);
  }
  // the key row: normed latent, rotated shared part
  long long slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
    slot = -1;
  }
  const T* row = dkv + (long long)t * dkv_stride;
  float acc = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_f32(row[c]);
    acc += v * v;
  }
  const float rstd = 1.f / sqrtf(block_sum(acc, scratch) / (float)rank + eps);
  if (slot < 0) return;
  T* dst = k_pages + slot * kw;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32(row[c]) * rstd * w_c[c]);
  for (int c = threadIdx.x; c < rot; c += blockDim.x) {
    float v = to_f32(row[rank + c]);
    if (c < rot_dims) {
      const bool second = interleaved ? (c & 1) : (c >= half);
      const int pc = interleaved ? (c ^ 1) : (second ? c - half : c + half);
      const int fi = interleaved ? (c >> 1) : (second ? c - half : c);
      const float sn = sn_s[fi], cs = cs_s[fi];
      const float other = to_f32(row[rank + pc]);
      v = second ? v * cs + other * sn : v * cs - other * sn;
    }
    dst[rank + c] = from_f32<T>(v);
  }
}

// One block per token.  qkv [tokens][stride]: q (num_q heads of head_dim) | k (num_kv heads of head_dim) | v (num_kv
// heads of v_dim) as projected; q_out [tokens][num_q * head_dim].
template <typename T>
__global__ void qkv_rows_prepare_kernel(const T* __restrict__ qkv, long long stride, T* __restrict__ q_out, int num_q,
                                        int num_kv, int head_dim, int v_dim, const float* __restrict__ wq,
                                        const float* __restrict__ wk, float eps, const float* __restrict__ inv_freq,
                                        int rot_dims, int interleaved, const int* __restrict__ positions,
                                        const float* __restrict__ q_head_scale, int v_unit,
                                        const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                        T* __restrict__ v_pages, long long num_slots, int* status) {
  __shared__ float scratch[33];
  __shared__ float cs_s[ROWS_MAX_ROT / 2], sn_s[ROWS_MAX_ROT / 2];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int q_size = num_q * head_dim, k_size = num_kv * head_dim, v_size = num_kv * v_dim;
  const T* q = qkv + (long long)t * stride;
  const T* k = q + q_size;
  const T* v = k + k_size;
  long long slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
    slot = -1;
  }
  const int half = rot_dims >> 1;
  if (rot_dims > 0) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &sn_s[i], &cs_s[i]);
  }
  float rq = 1.f, rk = 1.f;
  if (wq != nullptr) {
    float acc = 0.f;
    for (int c = threadIdx.x; c < q_size; c += blockDim.x) {
      const float x = to_f32(q[c]);
      acc += x * x;
    }
    rq = 1.f / sqrtf(block_sum(acc, scratch) / (float)q_size + eps);
    acc = 0.f;
    for (int c = threadIdx.x; c < k_size; c += blockDim.x) {
      const float x = to_f32(k[c]);
      acc += x * x;
    }
    rk = 1.f / sqrtf(block_sum(acc, scratch) / (float)k_size + eps);
  } else {
    __syncthreads();  // (the angles)
  }
  // q and k: norm, rotation, (q) the head's factor
  for (int c = threadIdx.x; c < q_size + k_size; c += blockDim.x) {
    const bool is_q = c < q_size;
    const int cc = is_q ? c : c - q_size;
    const T* src = is_q ? q : k;
    const float* w = is_q ? wq : wk;
    const float r = is_q ? rq : rk;
    const int h = cc / head_dim, j = cc - h * head_dim;
    float x = to_f32(src[cc]) * r * (w != nullptr ? w[cc] : 1.f);
    if (j < rot_dims) {
      const bool second = interleaved ? (j & 1) : (j >= half);
      const int pj = interleaved ? (j ^ 1) : (second ? j - half : j + half);
      const int fi = interleaved ? (j >> 1) : (second ? j - half : j);
      const int pc = h * head_dim + pj;
      const float other = to_f32(src[pc]) * r * (w != nullptr ? w[pc] : 1.f);
      x = second ? x * cs_s[fi] + other * sn_s[fi] : x * cs_s[fi] - other * sn_s[fi];
    }
    if (is_q) {
      if (q_head_scale != nullptr) x *= q_head_scale[h];
      q_out[(long long)t * q_size + cc] = from_f32<T>(x);
    } else if (slot >= 0) {
      k_pages[slot * k_size + cc] = from_f32<T>(x);
    }
  }
  if (slot < 0) return;
  // v: a warp per value head
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int g = warp; g < num_kv; g += warps) {
    const T* src = v + g * v_dim;
    float r = 1.f;
    if (v_unit) {
      float acc = 0.f;
      for (int j = lane; j < v_dim; j += 32) {
        const float x = to_f32(src[j]);
        acc += x * x;
      }
      r = 1.f / sqrtf(warp_sum(acc) / (float)v_dim + eps);
    }
    for (int j = lane; j < v_dim; j += 32) v_pages[slot * v_size + g * v_dim + j] = from_f32<T>(to_f32(src[j]) * r);
  }
}

// Two neighbouring elements in one store (the pair starts at an even element of a 4-byte aligned row: q_size,
// k_size and the channel are even, the buffers come from the allocator).
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
__device__ __forceinline__ void store_pair(__half* p, float a, float b) {
  *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}

// The same work with the token's row staged once in shared memory as 32-bit values (16-byte loads where the rows
// allow), the sums of squares formed while it is staged, and q and k handled two neighbouring channels at a time
// (a rotation of neighbours then needs no second read; paired stores).  Needs an even head size; `row` holds
// q | k | v.
template <typename T>
__global__ void qkv_rows_prepare_staged_kernel(const T* __restrict__ qkv, long long stride, T* __restrict__ q_out,
                                               int num_q, int num_kv, int head_dim, int v_dim,
                                               const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                               const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                                               const int* __restrict__ positions,
                                               const float* __restrict__ q_head_scale, int v_unit,
                                               const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                               T* __restrict__ v_pages, long long num_slots, int wide, int* status) {
  extern __shared__ __align__(16) float prep_row[];
  __shared__ float scratch2[64];
  __shared__ float cs_s[ROWS_MAX_ROT / 2], sn_s[ROWS_MAX_ROT / 2];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VEC = 16 / (int)sizeof(T);
  const int t = blockIdx.x;
  const int q_size = num_q * head_dim, k_size = num_kv * head_dim, v_size = num_kv * v_dim;
  const int width = q_size + k_size + v_size;
  const T* src = qkv + (long long)t * stride;
  long long slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
    slot = -1;
  }
  const int half = rot_dims >> 1;
  if (rot_dims > 0) {
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &sn_s[i], &cs_s[i]);
  }
  float acc_q = 0.f, acc_k = 0.f;
  if (wide) {  // (q_size and k_size are multiples of VEC: a piece lies in one of the three parts)
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      const T* e = reinterpret_cast<const T*>(&raw);
      float xs[VEC];
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        xs[i] = to_f32(e[i]);
        sq += xs[i] * xs[i];
      }
#pragma unroll
      for (int i = 0; i < VEC; i += 4)  // (c is a multiple of VEC, the array 16-byte aligned)
        *reinterpret_cast<float4*>(prep_row + c + i) = make_float4(xs[i], xs[i + 1], xs[i + 2], xs[i + 3]);
      if (c < q_size) acc_q += sq;
      else if (c < q_size + k_size) acc_k += sq;
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float x = to_f32(src[c]);
      prep_row[c] = x;
      if (c < q_size) acc_q += x * x;
      else if (c < q_size + k_size) acc_k += x * x;
    }
  }
  float rq = 1.f, rk = 1.f;
  if (wq != nullptr) {
    // both sums in one set of barriers (the order of additions depends only on the block's size)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    acc_q = warp_sum(acc_q);
    acc_k = warp_sum(acc_k);
    if (lane == 0) {
      scratch2[warp] = acc_q;
      scratch2[32 + warp] = acc_k;
    }
    __syncthreads();
    float tq = lane < nwarps ? scratch2[lane] : 0.f, tk = lane < nwarps ? scratch2[32 + lane] : 0.f;
    tq = warp_sum(tq);
    tk = warp_sum(tk);
    rq = 1.f / sqrtf(tq / (float)q_size + eps);
    rk = 1.f / sqrtf(tk / (float)k_size + eps);
  } else {
    __syncthreads();
  }
  const float inv_head_dim = 1.f / (float)head_dim;
  // q and k, two neighbouring channels per thread
  for (int c = threadIdx.x * 2; c < q_size + k_size; c += blockDim.x * 2) {
    const bool is_q = c < q_size;
    const int cc = is_q ? c : c - q_size;
    const float* w = is_q ? wq : wk;
    const float r = is_q ? rq : rk;
    // (the head by a product: (cc + 1/2) / head_dim is at least 1 / (2 head_dim) away from a whole number)
    const int h = __float2int_rd(((float)cc + 0.5f) * inv_head_dim), j = cc - h * head_dim;  // (j even, j + 1 in the head)
    const float2 xr = *reinterpret_cast<const float2*>(prep_row + c);
    float x0 = xr.x * r, x1 = xr.y * r;
    if (w != nullptr) {
      const float2 ww = *reinterpret_cast<const float2*>(w + cc);  // (cc is even, the weights 8-byte aligned)
      x0 *= ww.x;
      x1 *= ww.y;
    }
    if (j < rot_dims) {
      if (interleaved) {
        const float cs = cs_s[j >> 1], sn = sn_s[j >> 1];
        const float a = x0 * cs - x1 * sn, b = x1 * cs + x0 * sn;
        x0 = a;
        x1 = b;
      } else {
        // (rot_dims / 2 may be odd: the two channels are looked at one by one)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int ji = j + i;
          if (ji >= rot_dims) continue;
          const bool second = ji >= half;
          const int pj = second ? ji - half : ji + half, fi = second ? ji - half : ji;
          const int pc = c - j + pj;
          float other = prep_row[pc] * r;
          if (w != nullptr) other *= w[cc - j + pj];
          float& x = i ? x1 : x0;
          x = second ? x * cs_s[fi] + other * sn_s[fi] : x * cs_s[fi] - other * sn_s[fi];
        }
      }
    }
    if (is_q) {
      if (q_head_scale != nullptr) {
        x0 *= q_head_scale[h];
        x1 *= q_head_scale[h];
      }
      store_pair(q_out + (long long)t * q_size + cc, x0, x1);
    } else if (slot >= 0) {
      store_pair(k_pages + slot * k_size + cc, x0, x1);
    }
  }
  if (slot < 0) return;
  // v: a warp per value head
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* v = prep_row + q_size + k_size;
  for (int g = warp; g < num_kv; g += warps) {
    const float* vs = v + g * v_dim;
    float r = 1.f;
    if (v_unit) {
      float acc = 0.f;
      for (int j = lane; j < v_dim; j += 32) acc += vs[j] * vs[j];
      r = 1.f / sqrtf(warp_sum(acc) / (float)v_dim + eps);
    }
    for (int j = lane; j < v_dim; j += 32) v_pages[slot * v_size + g * v_dim + j] = from_f32<T>(vs[j] * r);
  }
}

static inline int prep_threads(int cols) {
  int threads = 32;
  while (threads < 256 && threads * 2 < cols) threads <<= 1;
  return threads;
}

// `wq` / `wk` null: no norm.  `v_pages` null: only the key pages are written.  `slot_mapping` null: nothing is stored.
extern "C" int ullm_kv_shared_prepare(int dtype, void* qk, long long stride, int tokens, int q_size, int kv_size,
                                      const float* wq, const float* wk, float eps, const int* slot_mapping,
                                      void* k_pages, void* v_pages, long long num_slots, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || q_size <= 0 || kv_size <= 0 || stride < q_size + kv_size) return ULLM_ERR_BAD_SIZE;
  if ((wq == nullptr) != (wk == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const dim3 grid(tokens), block(prep_threads(q_size));
#define KSP_GO(T)                                                                                                  \
  return ullm_launch_kernel(kv_shared_prepare_kernel<T>, grid, block, 0, st, (T*)qk, stride, q_size, kv_size, wq, wk, \
                            eps, slot_mapping, (T*)k_pages, (T*)v_pages, num_slots, status)
  if (dtype == ULLM_DTYPE_F32) KSP_GO(float);
  if (dtype == ULLM_DTYPE_BF16) KSP_GO(__nv_bfloat16);
  if (dtype == ULLM_DTYPE_F16) KSP_GO(__half);
#undef KSP_GO
  return ULLM_ERR_BAD_DTYPE;
}

// `v_pages` / `pv_pages` null: the values are the keys (one pooled row serves both).
extern "C" int ullm_pool_blocks(int dtype, const int* positions, const int* token_req, const int* req_slots,
                                const int* block_table, int max_pages, int page_size, long long num_pages,
                                const void* k_pages, const void* v_pages, int row, int v_row, const int* pool_slots,
                                long long num_pool_slots, void* pk_pages, void* pv_pages, int pool, int tokens,
                                int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || row <= 0 || pool <= 0 || page_size <= 0 || max_pages <= 0) return ULLM_ERR_BAD_SIZE;
  if ((v_pages == nullptr) != (pv_pages == nullptr) || (v_pages != nullptr && v_row <= 0)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const dim3 grid(tokens), block(prep_threads(row));
#define PB_GO(T)                                                                                                    \
  return ullm_launch_kernel(pool_blocks_kernel<T>, grid, block, 0, st, positions, token_req, req_slots, block_table, \
                            max_pages, page_size, num_pages, (const T*)k_pages, (const T*)v_pages, row, v_row,       \
                            pool_slots, num_pool_slots, (T*)pk_pages, (T*)pv_pages, pool, status)
  if (dtype == ULLM_DTYPE_F32) PB_GO(float);
  if (dtype == ULLM_DTYPE_BF16) PB_GO(__nv_bfloat16);
  if (dtype == ULLM_DTYPE_F16) PB_GO(__half);
#undef PB_GO
  return ULLM_ERR_BAD_DTYPE;
}

// `q_stride` / `dkv_stride`: elements between two tokens' rows of q_full / dkv (0: dense rows).
extern "C" int ullm_latent_prepare(int dtype, const void* q_full, const void* q_lat, const void* dkv, void* q_out,
                                   int tokens, int heads, int dim, int rot, int rank, int rot_dims, const float* w_c,
                                   float eps, const float* inv_freq, const int* positions, const int* slot_mapping,
                                   void* k_pages, long long num_slots, int* status, void* stream, int interleaved,
                                   long long q_stride, long long dkv_stride) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || heads <= 0 || dim <= 0 || rot < 0 || rank <= 0) return ULLM_ERR_BAD_SIZE;
  if (q_stride == 0) q_stride = (long long)heads * (dim + rot);
  if (dkv_stride == 0) dkv_stride = rank + rot;
  if (q_stride < (long long)heads * (dim + rot) || dkv_stride < rank + rot) return ULLM_ERR_BAD_SIZE;
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2 || (rot_dims > 0 && inv_freq == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (rot_dims > ROWS_MAX_ROT) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const dim3 grid(tokens), block(prep_threads(heads * rank / 4));
#define LP_GO(T)                                                                                                  \
  return ullm_launch_kernel(latent_prepare_kernel<T>, grid, block, 0, st, (const T*)q_full, q_stride,              \
                            (const T*)q_lat, (const T*)dkv, dkv_stride, (T*)q_out, tokens, heads, dim, rot, rank, rot_dims, interleaved, w_c, eps,  \
                            inv_freq, positions, slot_mapping, (T*)k_pages, num_slots, status)
  if (dtype == ULLM_DTYPE_F32) LP_GO(float);
  if (dtype == ULLM_DTYPE_BF16) LP_GO(__nv_bfloat16);
  if (dtype == ULLM_DTYPE_F16) LP_GO(__half);
#undef LP_GO
  return ULLM_ERR_BAD_DTYPE;
}

// `wq` / `wk` null: no norm of q and k.  `rot_dims` 0: no rotation.  `q_head_scale` null: none.  `slot_mapping` null:
// nothing is stored (q is still prepared).
extern "C" int ullm_qkv_rows_prepare(int dtype, const void* qkv, long long stride, void* q_out, int tokens, int num_q,
                                     int num_kv, int head_dim, int v_dim, const float* wq, const float* wk, float eps,
                                     const float* inv_freq, int rot_dims, int interleaved, const int* positions,
                                     const float* q_head_scale, int v_unit, const int* slot_mapping, void* k_pages,
                                     void* v_pages, long long num_slots, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || v_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (stride < (long long)num_q * head_dim + (long long)num_kv * (head_dim + v_dim)) return ULLM_ERR_BAD_SIZE;
  if ((wq == nullptr) != (wk == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (rot_dims < 0 || rot_dims > head_dim || rot_dims % 2) return ULLM_ERR_BAD_SIZE;
  if (rot_dims > 0 && (inv_freq == nullptr || positions == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (rot_dims > ROWS_MAX_ROT) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const dim3 grid(tokens), block(prep_threads(num_q * head_dim / 4));
  const long long width = (long long)num_q * head_dim + (long long)num_kv * (head_dim + v_dim);
  const size_t smem = (size_t)width * sizeof(float);
  const bool pairs_ok = (((uintptr_t)wq | (uintptr_t)wk) % 8 == 0) &&
                        (((uintptr_t)q_out | (uintptr_t)k_pages) % 8 == 0);
  const dim3 staged_block(block.x);  // (128 threads, all blocks of a 2,048-token step resident at once: no faster)
  if (head_dim % 2 == 0 && smem <= 160 * 1024 && pairs_ok) {
    // the staged form: the row waits in shared memory
    const int esize = dtype == ULLM_DTYPE_F32 ? 4 : 2, vec = 16 / esize;
    const int wide = ((uintptr_t)qkv % 16 == 0) && stride % vec == 0 && (num_q * head_dim) % vec == 0 &&
                     (num_kv * head_dim) % vec == 0 && width % vec == 0;
#define QRS_GO(T)                                                                                                    \
  {                                                                                                                  \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(qkv_rows_prepare_staged_kernel<T>,                                  \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
      cudaGetLastError();                                                                                            \
      return ULLM_ERR_LAUNCH;                                                                                        \
    }                                                                                                                \
    return ullm_launch_kernel(qkv_rows_prepare_staged_kernel<T>, grid, staged_block, smem, st, (const T*)qkv, stride, \
                              (T*)q_out, num_q, num_kv, head_dim, v_dim, wq, wk, eps, inv_freq, rot_dims,            \
                              interleaved, positions, q_head_scale, v_unit, slot_mapping, (T*)k_pages, (T*)v_pages,  \
                              num_slots, wide, status);                                                              \
  }
    if (dtype == ULLM_DTYPE_F32) QRS_GO(float);
    if (dtype == ULLM_DTYPE_BF16) QRS_GO(__nv_bfloat16);
    if (dtype == ULLM_DTYPE_F16) QRS_GO(__half);
#undef QRS_GO
    return ULLM_ERR_BAD_DTYPE;
  }
#define QRP_GO(T)                                                                                                    \
  return ullm_launch_kernel(qkv_rows_prepare_kernel<T>, grid, block, 0, st, (const T*)qkv, stride, (T*)q_out, num_q,  \
                            num_kv, head_dim, v_dim, wq, wk, eps, inv_freq, rot_dims, interleaved, positions,         \
                            q_head_scale, v_unit, slot_mapping, (T*)k_pages, (T*)v_pages, num_slots, status)
  if (dtype == ULLM_DTYPE_F32) QRP_GO(float);
  if (dtype == ULLM_DTYPE_BF16) QRP_GO(__nv_bfloat16);
  if (dtype == ULLM_DTYPE_F16) QRP_GO(__half);
#undef QRP_GO
  return ULLM_ERR_BAD_DTYPE;
}
