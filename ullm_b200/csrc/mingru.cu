// minGRU: a gated recurrence per channel whose gates read only the current token,
//
//   z_t = sigmoid(a_t + b_z)        u_t = x_t + b_x        c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t                       out_t = scale * S_t * silu(g_t)
//
// a | x | g are columns of ONE 32-bit product [tokens][stride]; the state S (32-bit, one row per request slot) is
// read at the start of a request's tokens of this step and written back behind them, so prompt portions of any
// length and single decoded tokens continue one another.  Everything is 32-bit; the output is rounded once.
//
// Two forms with the same arithmetic per token.  Few tokens per request (decode steps, short portions): one
// thread per (request, channel) walks the request's tokens in order.  Long portions: the recurrence is linear in S
// (S_t = A_t S_{t-1} + B_t), so a request's tokens are cut into chunks of MG_CHUNK; a first kernel folds each chunk
// into its (product of the A, B accumulated from zero), a second walks the chunks' pairs in order to get the
// state at each chunk's start (and the final state), a third replays each chunk from its start state and
// writes the outputs.  The chunks' cutting depends only on the token's place in the STEP's portion, so results
// differ from the walk by rounding only.
#include "common.cuh"

#define MG_THREADS 128
#define MG_CHUNK 64

__device__ __forceinline__ void mg_gates(float a, float x, float bz, float bx, float* z, float* c) {
  *z = 1.f / (1.f + expf(-(a + bz)));
  const float u = x + bx;
  *c = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
}

template <typename T>
__global__ void mingru_walk_kernel(const float* __restrict__ azg, long long stride, int a_off, int x_off, int g_off,
                                   const float* __restrict__ bz, const float* __restrict__ bx,
                                   float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                                   const int* __restrict__ req_slots, const int* __restrict__ token_req,
                                   T* __restrict__ out, long long out_stride, float out_scale, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (ch >= width) return;
  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  if (t1 <= t0) return;
  if (token_req[t0] < 0) {  // rows that belong to no request
    for (int t = t0; t < t1; ++t) out[(long long)t * out_stride + ch] = from_f32<T>(0.f);
    return;
  }
  float* sp = state + (long long)req_slots[r] * state_stride + ch;
  float S = *sp;
  const float bzc = bz[ch], bxc = bx[ch];
  for (int t = t0; t < t1; ++t) {
    const float* row = azg + (long long)t * stride;
    float z, c;
    mg_gates(row[a_off + ch], row[x_off + ch], bzc, bxc, &z, &c);
    S = (1.f - z) * S + z * c;
    const float g = row[g_off + ch];
    out[(long long)t * out_stride + ch] = from_f32<T>(out_scale * S * (g / (1.f + expf(-g))));
  }
  *sp = S;
}

// chunk k of the step covers rows k * MG_CHUNK .. of the flat batch, cut at request borders by `chunk_req` /
// `chunk_first` / `chunk_last` computed here from cu_q: a chunk never spans two requests because the grid is
// (channels, chunks per request, requests) and a chunk beyond the request's length does nothing.
__global__ void mingru_fold_kernel(const float* __restrict__ azg, long long stride, int a_off, int x_off,
                                   const float* __restrict__ bz, const float* __restrict__ bx,
                                   const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                   float* __restrict__ fold_a, float* __restrict__ fold_b, int max_chunks, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y, r = blockIdx.z;
  if (ch >= width) return;
  const int t0 = cu_q[r] + k * MG_CHUNK, t1 = min(cu_q[r + 1], t0 + MG_CHUNK);
  if (t0 >= t1 || token_req[cu_q[r]] < 0) return;
  const float bzc = bz[ch], bxc = bx[ch];
  float A = 1.f, B = 0.f;
  for (int t = t0; t < t1; ++t) {
    const float* row = azg + (long long)t * stride;
    float z, c;
    mg_gates(row[a_off + ch], row[x_off + ch], bzc, bxc, &z, &c);
    A *= 1.f - z;
    B = (1.f - z) * B + z * c;
  }
  const long long i = ((long long)r * max_chunks + k) * width + ch;
  fold_a[i] = A;
  fold_b[i] = B;
}

// the state at the start of every chunk (left in fold_b's place), and the request's state behind the step
__global__ void mingru_carry_kernel(float* __restrict__ fold_a, float* __restrict__ fold_b,
                                    float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                                    const int* __restrict__ req_slots, const int* __restrict__ token_req,
                                    int max_chunks, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (ch >= width) return;
  const int n = cu_q[r + 1] - cu_q[r];
  if (n <= 0 || token_req[cu_q[r]] < 0) return;
  float* sp = state + (long long)req_slots[r] * state_stride + ch;
  float S = *sp;
  const int chunks = (n + MG_CHUNK - 1) / MG_CHUNK;
  for (int k = 0; k < chunks; ++k) {
    const long long i = ((long long)r * max_chunks + k) * width + ch;
    const float A = fold_a[i], B = fold_b[i];
    fold_b[i] = S;
    S = A * S + B;
  }
  *sp = S;
}

template <typename T>
__global__ void mingru_replay_kernel(const float* __restrict__ azg, long long stride, int a_off, int x_off, int g_off,
                                     const float* __restrict__ bz, const float* __restrict__ bx,
                                     const float* __restrict__ start, const int* __restrict__ cu_q,
                                     const int* __restrict__ token_req, T* __restrict__ out, long long out_stride,
                                     float out_scale, int max_chunks, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y, r = blockIdx.z;
  if (ch >= width) return;
  const int t0 = cu_q[r] + k * MG_CHUNK, t1 = min(cu_q[r + 1], t0 + MG_CHUNK);
  if (t0 >= t1) return;
  if (token_req[cu_q[r]] < 0) {
    for (int t = t0; t < t1; ++t) out[(long long)t * out_stride + ch] = from_f32<T>(0.f);
    return;
  }
  const float bzc = bz[ch], bxc = bx[ch];
  float S = start[((long long)r * max_chunks + k) * width + ch];
  for (int t = t0; t < t1; ++t) {
    const float* row = azg + (long long)t * stride;
    float z, c;
    mg_gates(row[a_off + ch], row[x_off + ch], bzc, bxc, &z, &c);
    S = (1.f - z) * S + z * c;
    const float g = row[g_off + ch];
    out[(long long)t * out_stride + ch] = from_f32<T>(out_scale * S * (g / (1.f + expf(-g))));
  }
}

extern "C" int ullm_mingru_chunk() { return MG_CHUNK; }

// `max_q`: the longest portion of the step (host knowledge; it sizes the grid of the chunked form).  `fold`:
// scratch of 2 x requests x ceil(max_q / chunk) x width floats for the chunked form, or null: the walk is taken.
extern "C" int ullm_mingru(int out_dtype, const float* azg, long long stride, int a_off, int x_off, int g_off,
                           const float* bz, const float* bx, float* state, long long state_stride, const int* cu_q,
                           const int* req_slots, const int* token_req, void* out, long long out_stride,
                           float out_scale, int requests, int width, int max_q, float* fold, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (requests < 0 || width <= 0 || max_q < 0 || stride <= 0 || out_stride < width || state_stride < width)
    return ULLM_ERR_BAD_SIZE;
  if (requests == 0 || max_q == 0) return ULLM_OK;
  const int cb = (width + MG_THREADS - 1) / MG_THREADS;
  if (fold == nullptr || max_q <= MG_CHUNK) {
    const dim3 grid(cb, requests), block(MG_THREADS);
#define MG_WALK(T)                                                                                                   \
  return ullm_launch_kernel(mingru_walk_kernel<T>, grid, block, 0, st, azg, stride, a_off, x_off, g_off, bz, bx, state, \
                            state_stride, cu_q, req_slots, token_req, (T*)out, out_stride, out_scale, width)
    if (out_dtype == ULLM_DTYPE_F32) MG_WALK(float);
    if (out_dtype == ULLM_DTYPE_BF16) MG_WALK(__nv_bfloat16);
    if (out_dtype == ULLM_DTYPE_F16) MG_WALK(__half);
#undef MG_WALK
    return ULLM_ERR_BAD_DTYPE;
  }
  const int chunks = (max_q + MG_CHUNK - 1) / MG_CHUNK;
  if (chunks > 65535 || requests > 65535) return ULLM_ERR_BAD_SIZE;
  float* fold_a = fold;
  float* fold_b = fold + (long long)requests * chunks * width;
  int rc = ullm_launch_kernel(mingru_fold_kernel, dim3(cb, chunks, requests), dim3(MG_THREADS), 0, st, azg, stride,
                              a_off, x_off, bz, bx, cu_q, token_req, fold_a, fold_b, chunks, width);
  if (rc != ULLM_OK) return rc;
  rc = ullm_launch_kernel(mingru_carry_kernel, dim3(cb, requests), dim3(MG_THREADS), 0, st, fold_a, fold_b, state,
                          state_stride, cu_q, req_slots, token_req, chunks, width);
  if (rc != ULLM_OK) return rc;
  const dim3 grid(cb, chunks, requests), block(MG_THREADS);
#define MG_REPLAY(T)                                                                                                  \
  return ullm_launch_kernel(mingru_replay_kernel<T>, grid, block, 0, st, azg, stride, a_off, x_off, g_off, bz, bx,    \
                            (const float*)fold_b, cu_q, token_req, (T*)out, out_stride, out_scale, chunks, width)
  if (out_dtype == ULLM_DTYPE_F32) MG_REPLAY(float);
  if (out_dtype == ULLM_DTYPE_BF16) MG_REPLAY(__nv_bfloat16);
  if (out_dtype == ULLM_DTYPE_F16) MG_REPLAY(__half);
#undef MG_REPLAY
  return ULLM_ERR_BAD_DTYPE;
}
