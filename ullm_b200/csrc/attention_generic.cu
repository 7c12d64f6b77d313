// Paged causal attention for any mix of requests in one flat batch: prompt
// portions of any length beside single decoded tokens.  This is the general
// kernel: any head size up to 512 (key rows up to 640 where the values are a
// narrower part of them), any head counts, any page size, optional
// sliding window, float32 or bfloat16 storage.  It is the whole attention of
// the 32-bit path and the fallback of the bfloat16 path for sizes its
// tensor-core kernels do not take.
//
// One warp per (token, query head).  The query (scaled dot products in 32-bit)
// meets the keys 32 at a time, one key per lane; the running maximum, the
// running sum and the output accumulator are 32-bit (online softmax); exp is
// expf.  A token's keys are visited from the first visible position upward in
// groups of 32 counted from that position, so the result for a token does not
// depend on how the batch was cut, on the other requests in it, or on which
// pages hold the keys.
//
// Batch row r reads row req_slots[r] of the block table.  Request r owns query rows cu_q[r] .. cu_q[r+1]-1 and holds kv_len[r] tokens
// after this step; row j of it sits at position kv_len[r] - q_len[r] + j and
// sees positions max(0, pos - window + 1) .. pos (window 0 = all), and with
// `keep_first` > 0 also the positions below keep_first that the window has
// left behind (they are visited first, in groups of 32 of their own).
// Values may have a head size of their own (`v_dim`): the value pages are
// [*, page, kv heads, v_dim] and the output rows [heads, v_dim].
#include "common.cuh"

#define ATT_MAX_HEAD_DIM 512
#define ATT_MAX_KEY_DIM 640  // key rows that carry more than a head's values (a latent and a rotated part)
#define ATT_WARPS 4
#define ATT_O_REGS (ATT_MAX_HEAD_DIM / 32)

// Further options, all off in a zeroed struct.
//   slopes        [heads] 32-bit: the score of (query at position i, key at position j) loses slopes[h] * (i - j)
//   v_row, v_head elements between the value rows of two slots and between two value heads inside a row, for
//                 values that are a part of the KEY rows (v_cache = k_cache, v_row = kv heads x head_dim,
//                 v_head = head_dim: a head's values are the first v_dim elements of its key); 0: rows of their own
//   pool          P > 0: behind the window a query also sees ONE key / value per block of P positions that lies
//                 wholly before the window (block b = positions bP .. bP + P - 1, seen when bP + P - 1 <= i - window);
//                 entry b of the request sits in the pooled pages pk / pv ([*, page, kv heads, head_dim / v_dim],
//                 pv null: the first v_dim elements of pk's rows) through a block table of their own; they are
//                 visited first, in groups of 32 of their own, and share the softmax
//   gate          [tokens][heads x v_dim] (row stride gate_stride): out *= sigmoid(gate) before the one rounding
//   out_scale     multiplies the output (0 = 1); out_stride: elements between output rows (0: heads x v_dim)
struct AttExtras {
  const float* slopes;
  long long v_row, v_head;
  int pool;
  const void* pk;
  const void* pv;
  const int* p_block_table;
  int p_max_pages;
  long long p_num_pages;
  const void* gate;
  long long gate_stride;
  float out_scale;
  long long out_stride;
};

template <typename T, int OREGS>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, long long q_row_stride, T* __restrict__ out,
                                               const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                               const int* __restrict__ block_table, int max_pages,
                                               const int* __restrict__ req_slots,
                                               const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                                               const int* __restrict__ token_req, int tokens, int num_q, int num_kv,
                                               int head_dim, int page_size, int window, float scale,
                                               long long num_pages, int* status, int v_dim, int keep_first,
                                               float softcap, int v_rep, float* __restrict__ out_f32, AttExtras ex) {
  __shared__ float qs[ATT_WARPS][ATT_MAX_KEY_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * ATT_WARPS + warp;
  // v_rep == 1: one unit per (token, query head), which reads the values of its own kv head.  v_rep == num_kv:
  // a unit per (token, query head, VALUE head): head h's softmax weights applied to every kv head's values
  // (what mixing the weights across heads needs); the results are 32-bit rows [token][head][value head].
  const int units_per_token = num_q * v_rep;
  if (unit >= (long long)tokens * units_per_token) return;
  const int t = (int)(unit / units_per_token);
  const int hu = (int)(unit - (long long)t * units_per_token);
  const int h = hu / v_rep;
  const int kh = h / (num_q / num_kv);
  const int vh = v_rep > 1 ? hu - h * v_rep : kh;
  const long long out_row = ex.out_stride > 0 ? ex.out_stride : (long long)units_per_token * v_dim;
  T* o_ptr = out_f32 == nullptr ? out + (long long)t * out_row + (long long)hu * v_dim : nullptr;
  float* o32 = out_f32 != nullptr ? out_f32 + ((long long)t * units_per_token + hu) * v_dim : nullptr;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int r = token_req[t];
  const int q_len = r >= 0 ? cu_q[r + 1] - cu_q[r] : 0;
  const int kvl = r >= 0 ? kv_len[r] : 0;
  const int pos = kvl - q_len + (r >= 0 ? t - cu_q[r] : 0);
  if (r < 0 || q_len <= 0 || kvl <= 0 || pos < 0) {  // padding row
    for (int e = lane; e < v_dim; e += 32) {
      if (o32 != nullptr) o32[e] = 0.f;
      else o_ptr[e] = from_f32<T>(0.f);
    }
    return;
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const T* q_ptr = q + (long long)t * q_row_stride + (long long)h * head_dim;
  float* qv = qs[warp];
  for (int e = lane; e < head_dim; e += 32) qv[e] = to_f32(q_ptr[e]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[OREGS];
#pragma unroll
  for (int i = 0; i < OREGS; ++i) acc[i] = 0.f;
  const int* bt = block_table + (long long)req_slots[r] * max_pages;
  const long long kv_row = (long long)num_kv * head_dim;
  const long long v_row = ex.v_row > 0 ? ex.v_row : (long long)num_kv * v_dim;
  const long long v_head = ex.v_head > 0 ? ex.v_head : (long long)v_dim;
  const float slope = ex.slopes != nullptr ? ex.slopes[h] : 0.f;
  // three stretches of keys: the pooled blocks that lie wholly before the window, the kept first positions that
  // lie below the window, then the window
  const int kept = min(keep_first, lo);
  const int pooled = ex.pool > 0 ? lo / ex.pool : 0;
  const int* pbt = pooled > 0 ? ex.p_block_table + (long long)req_slots[r] * ex.p_max_pages : nullptr;
  const bool pv_own = ex.pv != nullptr;
  for (int part = pooled > 0 ? -1 : (kept > 0 ? 0 : 1); part < 2; ++part) {
  if (part == 0 && kept <= 0) continue;
  const int first = part == 1 ? lo : 0, last = part < 0 ? pooled - 1 : (part == 0 ? kept - 1 : pos);
  const T* kc = part < 0 ? (const T*)ex.pk : k_cache;
  const T* vc = part < 0 ? (pv_own ? (const T*)ex.pv : (const T*)ex.pk) : v_cache;
  const long long vr = part < 0 ? (pv_own ? (long long)num_kv * v_dim : kv_row) : v_row;
  const long long vhd = part < 0 ? (pv_own ? (long long)v_dim : (long long)head_dim) : v_head;
  const int* tab = part < 0 ? pbt : bt;
  const long long pages_here = part < 0 ? ex.p_num_pages : num_pages;
  for (int base = first; base <= last; base += 32) {
    const int key = base + lane;
    const bool valid = key <= last;
    long long slot = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = tab[key / page_size];
      if (page < 0 || page >= pages_here) {
        ullm_report(status, ULLM_STATUS_PAGE, t, page);
      } else {
        slot = (long long)page * page_size + key % page_size;
        const T* kp = kc + slot * kv_row + (long long)kh * head_dim;
        float d = 0.f;
        for (int e = 0; e < head_dim; ++e) d += qv[e] * to_f32(kp[e]);
        s = d * scale;
        if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
        if (part >= 0) s -= slope * (float)(pos - key);
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (slot >= 0) ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);  // m = -inf on the first group: 0
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < OREGS; ++i) acc[i] *= alpha;
    const int n = min(32, last - base + 1);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long sj = __shfl_sync(0xffffffffu, slot, j);
      if (sj < 0) continue;
      const T* vp = vc + sj * vr + (long long)vh * vhd;
#pragma unroll
      for (int i = 0; i < OREGS; ++i) {
        const int e = lane + 32 * i;
        if (e < v_dim) acc[i] += pj * to_f32(vp[e]);
      }
    }
    m = m_new;
  }
  }
  const float inv = (l > 0.f ? 1.f / l : 0.f) * (ex.out_scale != 0.f ? ex.out_scale : 1.f);
  const T* gate = ex.gate != nullptr ? (const T*)ex.gate + (long long)t * ex.gate_stride + (long long)hu * v_dim : nullptr;
#pragma unroll
  for (int i = 0; i < OREGS; ++i) {
    const int e = lane + 32 * i;
    if (e < v_dim) {
      float o = acc[i] * inv;
      if (gate != nullptr) o /= 1.f + expf(-to_f32(gate[e]));
      if (o32 != nullptr) o32[e] = o;
      else o_ptr[e] = from_f32<T>(o);
    }
  }
}

// Softmax weights mixed across heads, w'_h = sum_g M[h][g] w_g, applied to head h's own values:
// out[t][h] = sum_g M[h][g] * part[t][g][kv head of h], with part = every head's weights applied to every kv
// head's values (32-bit, from the kernel above with v_rep = num_kv).  One thread per (token, kv head, element)
// reads its column of the parts once and finishes the GQ heads of that kv head together; the mixer lies in shared
// memory.  GQ = 0: any group size, one head at a time.
template <typename T, int GQ>
__global__ void mix_heads_kernel(const float* __restrict__ part, const float* __restrict__ mix, T* __restrict__ out,
                                 long long total, int num_q, int num_kv, int v_dim, int in_smem) {
  extern __shared__ float mix_smem[];  // [num_q][num_q], unless the mixer is too large for it
  pdl_launch_dependents();
  pdl_wait();
  if (in_smem) {
    for (int i = threadIdx.x; i < num_q * num_q; i += blockDim.x) mix_smem[i] = mix[i];
    __syncthreads();
  }
  const float* mix_s = in_smem ? mix_smem : mix;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int e = (int)(i % v_dim);
  const long long tc = i / v_dim;
  const int c = (int)(tc % num_kv);
  const long long t = tc / num_kv;
  const int gq = num_q / num_kv;
  const float* p = part + ((t * num_q) * num_kv + c) * v_dim + e;
  const long long step = (long long)num_kv * v_dim;
  T* o = out + (t * num_q + (long long)c * gq) * v_dim + e;
  if (GQ > 0) {
    float acc[GQ > 0 ? GQ : 1];
#pragma unroll
    for (int j = 0; j < GQ; ++j) acc[j] = 0.f;
    for (int g = 0; g < num_q; ++g) {
      const float pv = p[g * step];
#pragma unroll
      for (int j = 0; j < GQ; ++j) acc[j] = fmaf(mix_s[(c * GQ + j) * num_q + g], pv, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < GQ; ++j) o[(long long)j * v_dim] = from_f32<T>(acc[j]);
  } else {
    for (int j = 0; j < gq; ++j) {
      float acc = 0.f;
      for (int g = 0; g < num_q; ++g) acc = fmaf(mix_s[(c * gq + j) * num_q + g], p[g * step], acc);
      o[(long long)j * v_dim] = from_f32<T>(acc);
    }
  }
}

template <typename T>
static int launch_mix(const float* parts, const float* mix, void* out, int tokens, int num_q, int num_kv, int v_dim,
                      cudaStream_t st) {
  const long long total = (long long)tokens * num_kv * v_dim;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  const dim3 grid((int)blocks), block(256);
  size_t smem = (size_t)num_q * num_q * sizeof(float);
  const int in_smem = smem <= 40 * 1024;
  if (!in_smem) smem = 0;
#define MIX_GO(GQ)                                                                                                  \
  return ullm_launch_kernel(mix_heads_kernel<T, GQ>, grid, block, smem, st, parts, mix, (T*)out, total, num_q, num_kv, \
                            v_dim, in_smem)
  switch (num_q / num_kv) {
    case 1: MIX_GO(1);
    case 2: MIX_GO(2);
    case 4: MIX_GO(4);
    case 8: MIX_GO(8);
    default: MIX_GO(0);
  }
#undef MIX_GO
}

template <typename T>
static int launch_generic(const void* q, long long q_row_stride, void* out, const void* k_cache, const void* v_cache,
                          const int* block_table, int max_pages, const int* req_slots, const int* cu_q,
                          const int* kv_len, const int* token_req, int tokens, int num_q, int num_kv, int head_dim, int page_size,
                          int window, float scale, long long num_pages, int* status, cudaStream_t st, int v_dim,
                          int keep_first, float softcap = 0.f, int v_rep = 1, float* out_f32 = nullptr,
                          AttExtras ex = AttExtras{}) {
  const long long units = (long long)tokens * num_q * v_rep;
  const long long blocks = (units + ATT_WARPS - 1) / ATT_WARPS;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
#define LAUNCH(OREGS)                                                                                             \
  rc = ullm_launch_kernel(paged_attention_generic_kernel<T, OREGS>, dim3((int)blocks), dim3(ATT_WARPS * 32), 0, st, \
      (const T*)q, q_row_stride, (T*)out, (const T*)k_cache, (const T*)v_cache, block_table, max_pages, req_slots,  \
      cu_q, kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages, status,       \
      v_dim, keep_first, softcap, v_rep, out_f32, ex)
  int rc = ULLM_OK;
  if (v_dim <= 32) LAUNCH(1);
  else if (v_dim <= 64) LAUNCH(2);
  else if (v_dim <= 128) LAUNCH(4);
  else if (v_dim <= 256) LAUNCH(8);
  else LAUNCH(16);
#undef LAUNCH
  return rc;
}

// `v_dim`: head size of the values (and of the output); `keep_first`: positions below it stay visible;
// `softcap` > 0: score <- softcap * tanh(score / softcap); `out_parts` (32-bit, [tokens][heads][kv heads][v_dim])
// non-null: every head's weights are applied to EVERY kv head's values and left there unrounded (`out` unused),
// for `ullm_mix_heads`.
extern "C" int ullm_paged_attention_generic_ex2(int dtype, const void* q, long long q_row_stride, void* out,
                                                const void* k_cache, const void* v_cache, const int* block_table,
                                                int max_pages, const int* req_slots, const int* cu_q,
                                                const int* kv_len, const int* token_req, int tokens, int num_q,
                                                int num_kv, int head_dim, int page_size, int window, float scale,
                                                long long num_pages, int* status, void* stream, int v_dim,
                                                int keep_first, float softcap, float* out_parts) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || page_size <= 0 || max_pages <= 0)
    return ULLM_ERR_BAD_SIZE;
  if (num_q % num_kv != 0 || head_dim > ATT_MAX_HEAD_DIM || window < 0 || v_dim <= 0 || v_dim > ATT_MAX_HEAD_DIM ||
      keep_first < 0 || softcap < 0.f)
    return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const int v_rep = out_parts != nullptr ? num_kv : 1;
  if (dtype == ULLM_DTYPE_F32)
    return launch_generic<float>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                 kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                 status, st, v_dim, keep_first, softcap, v_rep, out_parts);
  if (dtype == ULLM_DTYPE_BF16)
    return launch_generic<__nv_bfloat16>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                         kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale,
                                         num_pages, status, st, v_dim, keep_first, softcap, v_rep, out_parts);
  if (dtype == ULLM_DTYPE_F16)
    return launch_generic<__half>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                  kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                  status, st, v_dim, keep_first, softcap, v_rep, out_parts);
  return ULLM_ERR_BAD_DTYPE;
}

// The general kernel with the further options of `AttExtras` (see there): distance slopes, values inside the key
// rows (`values_in_keys`), pooled blocks behind the window, an output gate, a scale and a row stride of the output.
extern "C" int ullm_paged_attention_generic_ex3(int dtype, const void* q, long long q_row_stride, void* out,
                                                const void* k_cache, const void* v_cache, const int* block_table,
                                                int max_pages, const int* req_slots, const int* cu_q,
                                                const int* kv_len, const int* token_req, int tokens, int num_q,
                                                int num_kv, int head_dim, int page_size, int window, float scale,
                                                long long num_pages, int* status, void* stream, int v_dim,
                                                int keep_first, float softcap, const float* slopes,
                                                int values_in_keys, int pool, const void* pk, const void* pv,
                                                const int* p_block_table, int p_max_pages, long long p_num_pages,
                                                const void* gate, long long gate_stride, float out_scale,
                                                long long out_stride) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || page_size <= 0 || max_pages <= 0)
    return ULLM_ERR_BAD_SIZE;
  if (num_q % num_kv != 0 || head_dim > ATT_MAX_KEY_DIM || window < 0 || v_dim <= 0 || v_dim > ATT_MAX_HEAD_DIM ||
      keep_first < 0 || softcap < 0.f || pool < 0)
    return ULLM_ERR_UNSUPPORTED;
  if (values_in_keys && v_dim > head_dim) return ULLM_ERR_BAD_SIZE;
  if (pool > 0 && (window <= 0 || pk == nullptr || p_block_table == nullptr || p_max_pages <= 0 || keep_first > 0 ||
                   slopes != nullptr))
    return ULLM_ERR_UNSUPPORTED;
  if (out_stride != 0 && out_stride < (long long)num_q * v_dim) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  AttExtras ex = {};
  ex.slopes = slopes;
  if (values_in_keys) {
    v_cache = k_cache;
    ex.v_row = (long long)num_kv * head_dim;
    ex.v_head = head_dim;
  }
  ex.pool = pool;
  ex.pk = pk;
  ex.pv = pv;
  ex.p_block_table = p_block_table;
  ex.p_max_pages = p_max_pages;
  ex.p_num_pages = p_num_pages;
  ex.gate = gate;
  ex.gate_stride = gate_stride;
  ex.out_scale = out_scale;
  ex.out_stride = out_stride;
  if (dtype == ULLM_DTYPE_F32)
    return launch_generic<float>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                 kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                 status, st, v_dim, keep_first, softcap, 1, nullptr, ex);
  if (dtype == ULLM_DTYPE_BF16)
    return launch_generic<__nv_bfloat16>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                         kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale,
                                         num_pages, status, st, v_dim, keep_first, softcap, 1, nullptr, ex);
  if (dtype == ULLM_DTYPE_F16)
    return launch_generic<__half>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                  kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                  status, st, v_dim, keep_first, softcap, 1, nullptr, ex);
  return ULLM_ERR_BAD_DTYPE;
}

// out [tokens][heads][v_dim] (the engine's dtype) = the parts mixed by `mix` [heads][heads] (32-bit).
extern "C" int ullm_mix_heads(int dtype, const float* parts, const float* mix, void* out, int tokens, int num_q,
                              int num_kv, int v_dim, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || v_dim <= 0 || num_q % num_kv) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  if (dtype == ULLM_DTYPE_F32) return launch_mix<float>(parts, mix, out, tokens, num_q, num_kv, v_dim, st);
  if (dtype == ULLM_DTYPE_BF16) return launch_mix<__nv_bfloat16>(parts, mix, out, tokens, num_q, num_kv, v_dim, st);
  if (dtype == ULLM_DTYPE_F16) return launch_mix<__half>(parts, mix, out, tokens, num_q, num_kv, v_dim, st);
  return ULLM_ERR_BAD_DTYPE;
}

// `v_dim`: head size of the values (and of the output); `keep_first`: positions below it stay visible.
extern "C" int ullm_paged_attention_generic_ex(int dtype, const void* q, long long q_row_stride, void* out,
                                               const void* k_cache, const void* v_cache, const int* block_table,
                                               int max_pages, const int* req_slots, const int* cu_q,
                                               const int* kv_len, const int* token_req, int tokens, int num_q,
                                               int num_kv, int head_dim, int page_size, int window, float scale,
                                               long long num_pages, int* status, void* stream, int v_dim,
                                               int keep_first) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || page_size <= 0 || max_pages <= 0)
    return ULLM_ERR_BAD_SIZE;
  if (num_q % num_kv != 0 || head_dim > ATT_MAX_HEAD_DIM || window < 0 || v_dim <= 0 || v_dim > ATT_MAX_HEAD_DIM ||
      keep_first < 0)
    return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  if (dtype == ULLM_DTYPE_F32)
    return launch_generic<float>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                 kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                 status, st, v_dim, keep_first);
  if (dtype == ULLM_DTYPE_BF16)
    return launch_generic<__nv_bfloat16>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                         kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale,
                                         num_pages, status, st, v_dim, keep_first);
  if (dtype == ULLM_DTYPE_F16)
    return launch_generic<__half>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                  kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                  status, st, v_dim, keep_first);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_paged_attention_generic(int dtype, const void* q, long long q_row_stride, void* out,
                                            const void* k_cache, const void* v_cache, const int* block_table,
                                            int max_pages, const int* req_slots, const int* cu_q, const int* kv_len,
                                            const int* token_req,
                                            int tokens, int num_q, int num_kv, int head_dim, int page_size, int window,
                                            float scale, long long num_pages, int* status, void* stream) {
  return ullm_paged_attention_generic_ex(dtype, q, q_row_stride, out, k_cache, v_cache, block_table, max_pages,
                                         req_slots, cu_q, kv_len, token_req, tokens, num_q, num_kv, head_dim,
                                         page_size, window, scale, num_pages, status, stream, head_dim, 0);
}
