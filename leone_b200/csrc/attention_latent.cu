// Attention through a cached latent (one key/value head shared by all query heads).
//
// Per token the cache row is [c (rank) | r (rot_dim)]: c is the RMS-normed latent, r one rotated
// key part shared by all heads.  A head's key is (W_uk c, r) and its value W_uv c; with the
// products moved to the query side (q_lat = W_uk^T q_plain, out = W_uv sum_j w_j c_j) the
// attention runs on the cache rows themselves:
//
//   score_j = (q_lat . c_j + q_rot . r_j) * scale,   o_lat = sum_j w_j c_j
//
// Softmax in fp32 over the keys lo..p of the query's own sequence (lo = 0, or p-window+1), with an
// optional per-head sink: exp(sink_h) joins the denominator once, without a key or a value.  An
// optional per-head output gate multiplies the head's result by sigmoid(gate[t, h]).
//
// `latent_prepare` makes the cache rows and the rotated query parts of a step's tokens:
// c = rms_norm(dkv[:rank]) * w, r = rotate(dkv[rank:]) into the page of (sequence, position);
// rotate(q_rot) of every head into the query buffer.  Angles are position * frequency_i, formed and
// evaluated in fp32; cos and sin are multiplied by `magnitude`.
#include "common.cuh"

namespace leone {

constexpr int kLatThreads = 128;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// rotate pair i of `src` (rot_dims leading elements rotate, the rest pass) into dst, all fp32 math
template <typename T>
__device__ __forceinline__ void rotate_into(const T* __restrict__ src, T* __restrict__ dst, int rot_dim,
                                            int rot_dims, const float* cs, int adjacent, int tid, int nthreads) {
  const int half = rot_dims / 2;
  for (int i = tid; i < half; i += nthreads) {
    const int a = adjacent ? 2 * i : i, b = adjacent ? 2 * i + 1 : i + half;
    const float u = to_float<T>(src[a]), v = to_float<T>(src[b]);
    const float c = cs[2 * i], s = cs[2 * i + 1];
    dst[a] = from_float<T>(u * c - v * s);
    dst[b] = from_float<T>(v * c + u * s);
  }
  for (int i = rot_dims + tid; i < rot_dim; i += nthreads) dst[i] = src[i];
}

template <typename T, typename TW>
__global__ void __launch_bounds__(kLatThreads)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int q_off, int dkv_off, T* __restrict__ q_abs,
                      int heads, int dim, int rot_dim, int rank, const TW* __restrict__ norm_w, float eps,
                      const float* __restrict__ freqs, int rot_dims, float magnitude, int adjacent,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ block_table, int table_width, int n_seqs, T* __restrict__ pool,
                      int num_pages, int page_tokens, int* status) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  float* cs = smem;                 // [rot_dims/2][2]
  __shared__ float scratch[33];
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t], s = seq_of_token[t];
  const int half = rot_dims / 2;
  for (int i = tid; i < half; i += kLatThreads) {
    const float a = (float)pos * freqs[i];
    cs[2 * i] = cosf(a) * magnitude;
    cs[2 * i + 1] = sinf(a) * magnitude;
  }
  __syncthreads();
  const T* row = proj + (size_t)t * ld;
  const int dk = rank + rot_dim;
  // the query's rotated parts
  for (int h = 0; h < heads; ++h)
    rotate_into<T>(row + q_off + (size_t)h * (dim + rot_dim) + dim, q_abs + ((size_t)t * heads + h) * dk + rank,
                   rot_dim, rot_dims, cs, adjacent, tid, kLatThreads);
  if (pool == nullptr) return;
  if (s < 0 || s >= n_seqs || pos < 0) {
    if (tid == 0) set_status(status, s < 0 || s >= n_seqs ? kBadSequence : kBadPosition, t, pos);
    return;
  }
  const int blk = pos / page_tokens;
  const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
  if (page < 0 || page >= num_pages) {
    if (tid == 0) set_status(status, kBadPage, t, page);
    return;
  }
  T* dst = pool + ((size_t)page * page_tokens + (pos % page_tokens)) * dk;
  const T* dkv = row + dkv_off;
  float ss = 0.f;
  for (int c = tid; c < rank; c += kLatThreads) {
    const float x = to_float<T>(dkv[c]);
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)rank + eps);
  for (int c = tid; c < rank; c += kLatThreads)
    dst[c] = from_float<T>(to_float<T>(dkv[c]) * r * to_float<TW>(norm_w[c]));
  rotate_into<T>(dkv + rank, dst + rank, rot_dim, rot_dims, cs, adjacent, tid, kLatThreads);
}

// One block per (token, head).  q: [n, heads, dk] (latent part first); pool rows of dk elements,
// the first dv of which are the value; out: [n, heads, dv].
template <typename T, typename TS, int ACC>
__global__ void __launch_bounds__(kLatThreads)
attention_latent_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ pool,
                        const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions, int heads,
                        int dk, int dv, float scale, int window, const TS* __restrict__ sink,
                        const T* __restrict__ gate, int ldg, int page_tokens, int num_pages, int n_seqs,
                        int* status) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  long long* off_s = (long long*)smem;                // [128] row index into the pool
  float* p_s = smem + 2 * kLatThreads;                // [128]
  float* q_s = p_s + kLatThreads;                     // [dk]
  __shared__ float scratch[33];
  __shared__ int bad;
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t], s = seq_of_token[t];
  T* dst = out + ((size_t)t * heads + h) * dv;
  if (tid == 0) bad = 0;
  if (s < 0 || s >= n_seqs || pos < 0) {
    if (tid == 0) set_status(status, s < 0 || s >= n_seqs ? kBadSequence : kBadPosition, t, pos);
    for (int c = tid; c < dv; c += kLatThreads) dst[c] = from_float<T>(0.f);
    return;
  }
  const T* qr = q + ((size_t)t * heads + h) * dk;
  for (int c = tid; c < dk; c += kLatThreads) q_s[c] = to_float<T>(qr[c]);
  __syncthreads();
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // the sink is a score of its own: it joins the maximum and the denominator, nothing else
  float m_run = -INFINITY, l_run = 0.f;
  if (sink != nullptr) {
    m_run = to_float<TS>(sink[h]);
    l_run = 1.f;
  }
  float acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
  for (int j0 = lo; j0 <= pos; j0 += kLatThreads) {
    const int j = j0 + tid;
    float score = -INFINITY;
    long long row_index = -1;
    if (j <= pos) {
      const int blk = j / page_tokens;
      const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
      if (page < 0 || page >= num_pages) {
        set_status(status, kBadPage, t, page, j);
        bad = 1;
      } else {
        row_index = (long long)page * page_tokens + (j % page_tokens);
        const T* krow = pool + row_index * dk;
        float dot = 0.f;
        for (int c = 0; c < dk; ++c) dot = fmaf(q_s[c], to_float<T>(krow[c]), dot);
        score = dot * scale;
      }
    }
    off_s[tid] = row_index;
    const float tile_max = block_max(score, scratch);
    const float m_new = fmaxf(m_run, tile_max);
    const float p = (row_index >= 0) ? expf(score - m_new) : 0.f;
    p_s[tid] = p;
    const float tile_sum = block_sum(p, scratch);   // also orders the p_s/off_s writes before the reads
    const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int count = min(kLatThreads, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int c = tid + i * kLatThreads;
      if (c < dv) {
        float a = acc[i] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const long long r = off_s[jj];
          if (r >= 0) a = fmaf(p_s[jj], to_float<T>(pool[r * dk + c]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  float f = (l_run > 0.f && !bad) ? 1.f / l_run : 0.f;
  if (gate != nullptr) f *= sigmoidf_(to_float<T>(gate[(size_t)t * ldg + h]));
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int c = tid + i * kLatThreads;
    if (c < dv) dst[c] = from_float<T>(acc[i] * f);
  }
}

}  // namespace leone

using namespace leone;

extern "C" int leone_latent_prepare(int dtype, const void* proj, int ld, int q_off, int dkv_off, void* q_abs,
                                    int n_tokens, int heads, int dim, int rot_dim, int rank,
                                    const void* norm_w, int w_dtype, float eps, const float* freqs,
                                    int rot_dims, float magnitude, int adjacent, const int* positions,
                                    const int* seq_of_token, const int* block_table, int table_width,
                                    int n_seqs, void* pool, int num_pages, int page_tokens, int* status,
                                    cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || dim < 0 || rot_dim < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2)
    return kRefusedSize;
  if (pool != nullptr && (page_tokens <= 0 || table_width <= 0)) return kRefusedSize;
  const size_t smem = sizeof(float) * (size_t)(rot_dims + 2);
#define PREP(T, TW)                                                                                          \
  launch_kernel(latent_prepare_kernel<T, TW>, dim3(n_tokens), dim3(kLatThreads), smem, stream,                                      \
      (const T*)proj, ld, q_off, dkv_off, (T*)q_abs, heads, dim, rot_dim, rank, (const TW*)norm_w, eps,    \
      freqs, rot_dims, magnitude, adjacent, positions, seq_of_token, block_table, table_width, n_seqs,     \
      (T*)pool, num_pages, page_tokens, status)
  if (dtype == 0 && w_dtype == 0) PREP(float, float);
  else if (dtype == 1 && w_dtype == 0) PREP(__nv_bfloat16, float);
  else if (dtype == 1 && w_dtype == 1) PREP(__nv_bfloat16, __nv_bfloat16);
  else return kRefusedDtype;
#undef PREP
  return launch_result();
}

// sink: per head, in `sink_dtype` (0 fp32, 1 bfloat16), or null; gate: [n, >= heads] rows `ldg`
// apart in the run dtype, or null.
extern "C" int leone_attention_latent(int dtype, const void* q, void* out, const void* pool,
                                      const int* block_table, int table_width, const int* seq_of_token,
                                      const int* positions, int n_tokens, int heads, int dk, int dv,
                                      float scale, int window, const void* sink, int sink_dtype,
                                      const void* gate, int ldg, int page_tokens, int num_pages, int n_seqs,
                                      int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dv <= 0 || dv > dk || dv > kLatThreads * 8 || page_tokens <= 0 ||
      table_width <= 0)
    return kRefusedSize;
  const dim3 grid(n_tokens, heads);
  const size_t smem = (size_t)(dk + kLatThreads) * sizeof(float) + kLatThreads * sizeof(long long) + 8;
  if (smem > 48 * 1024) return kRefusedSize;
#define ATT(T, TS, A)                                                                                       \
  launch_kernel(attention_latent_kernel<T, TS, A>, grid, dim3(kLatThreads), smem, stream,                                    \
      (const T*)q, (T*)out, (const T*)pool, block_table, table_width, seq_of_token, positions, heads, dk, \
      dv, scale, window, (const TS*)sink, (const T*)gate, ldg, page_tokens, num_pages, n_seqs, status)
#define ATT_A(T, TS)                          \
  do {                                        \
    if (dv <= kLatThreads) ATT(T, TS, 1);     \
    else if (dv <= 2 * kLatThreads) ATT(T, TS, 2); \
    else if (dv <= 4 * kLatThreads) ATT(T, TS, 4); \
    else ATT(T, TS, 8);                       \
  } while (0)
  if (dtype == 0 && sink_dtype == 0) ATT_A(float, float);
  else if (dtype == 1 && sink_dtype == 0) ATT_A(__nv_bfloat16, float);
  else if (dtype == 1 && sink_dtype == 1) ATT_A(__nv_bfloat16, __nv_bfloat16);
  else return kRefusedDtype;
#undef ATT_A
#undef ATT
  return launch_result();
}
