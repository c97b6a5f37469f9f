// Linear attention with a decaying state per head (no softmax):
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S: [dim, vdim] fp32, per request and head
//   o_t = S_t^T q_t
//
// with q, k, v = silu(their projections).  The state is read from and written back to the
// request's state slot, so a sequence may be cut into steps anywhere: the recurrence is run token
// by token in the same order whatever the cut, and a step of one token per sequence (decode) is
// the same kernel.  Everything but the stored projections is fp32.
//
// Two forms:
//  * `scan`: one block per (value slice, head, sequence) walks the step's tokens of its sequence
//    in order.  The block's threads are (32 lanes of value columns) x (DP parts of the key
//    dimension); a thread keeps its rows of one or four state columns in registers.
//  * chunk-parallel (long prompt portions): a sequence's tokens are cut into chunks of `chunk`
//    tokens; (1) every chunk but the last sums its own k v^T contributions from a zero state,
//    (2) a pass over the chunks turns those into the state at each chunk's start
//    (S_c = decay^chunk * S_(c-1) + D_(c-1)) and writes the final state's predecessor, (3) every
//    chunk walks its tokens from its start state.  Same per-token arithmetic, 1.5 times the work,
//    parallel over chunks.
//
// Then `gate_norm`: the heads of a token, concatenated, are RMS-normed together (fp32), multiplied
// by a weight and by sigmoid(gate projection), and stored in the run dtype.
#include "common.cuh"

namespace leone {

constexpr int kVS = 32;        // value columns per block
constexpr int kTB = 16;        // tokens staged in shared memory at a time

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// mode 0: state from `chunk_state`/the slot, outputs written, final state to the slot (last chunk)
// mode 1: state from zero, no outputs, final state to `chunk_state` (a chunk's own contribution)
// A thread owns VPT value columns of DPT rows of the state, so a k or q element read from shared
// memory serves VPT multiply-adds.
template <typename T, int DPT, int VPT, bool OUT, bool FAST>
__global__ void __launch_bounds__(256, (DPT * VPT <= 64) ? 2 : 1)      // two blocks an SM where the state fits 128 registers
linear_attention_scan_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                             float* __restrict__ out, int ldo, float* state, float* chunk_state,
                             const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                             const float* __restrict__ decay, int heads, int dim, int vdim,
                             int chunk, int n_seqs, int n_slots, int* status) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  constexpr int mode = OUT ? 0 : 1;
  extern __shared__ __align__(16) float smem[];
  constexpr int VW = kVS * VPT;            // value columns per block
  const int DP = blockDim.y;
  float* q_s = smem;                       // [kTB][dim]
  float* k_s = q_s + kTB * dim;            // [kTB][dim]
  float* v_s = k_s + kTB * dim;            // [kTB][VW]
  float* part = v_s + kTB * VW;            // [DP][kTB][VW]
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int tid = ty * kVS + tx, nthreads = kVS * DP;
  const int h = blockIdx.y;
  int s = blockIdx.z, c = 0;
  const int v0 = blockIdx.x * VW;
  int t0, t1;
  if (chunk > 0) {
    // blockIdx.z counts (sequence, chunk) pairs: find this block's
    int z = blockIdx.z, b = 0;
    while (b < n_seqs) {
      const int len = q_start[b + 1] - q_start[b];
      const int nc = (len + chunk - 1) / chunk;
      if (z < nc) break;
      z -= nc;
      ++b;
    }
    if (b >= n_seqs) return;
    s = b;
    c = z;
    t0 = q_start[s] + c * chunk;
    t1 = min(q_start[s + 1], t0 + chunk);
    if (mode == 1 && t1 == q_start[s + 1]) return;      // the last chunk's contribution is never needed
  } else {
    t0 = q_start[s];
    t1 = q_start[s + 1];
  }
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) {
    if (tid == 0) set_status(status, kBadSequence, s, slot);
    return;
  }
  const float dec = decay[h];
  const int d_per = (dim + DP - 1) / DP;
  const int d0 = ty * d_per;
  const size_t per_head = (size_t)dim * vdim;
  // where this block's start state is, and where its end state goes
  const float* s_in = nullptr;
  float* s_out = nullptr;
  float* slot_state = state + ((size_t)slot * heads + h) * per_head;
  if (chunk > 0) {
    // chunk_state: [chunk pairs][heads][dim][vdim]; an entry holds (mode 1) its chunk's own
    // contribution, later (after the prefix pass) the state at the chunk's start
    float* mine = chunk_state + ((size_t)blockIdx.z * heads + h) * per_head;
    if (mode == 1) s_out = mine;
    else {
      s_in = mine;
      s_out = t1 == q_start[s + 1] ? slot_state : nullptr;
    }
  } else {
    s_in = slot_state;
    s_out = slot_state;
  }
  float S[DPT][VPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = d0 + i;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = v0 + j * kVS + tx;
      S[i][j] = (s_in != nullptr && i < d_per && d < dim && v < vdim) ? s_in[(size_t)d * vdim + v] : 0.f;
    }
  }
  // FAST (bfloat16, 16-byte aligned rows, one 8-element piece of q, k and v per thread and batch):
  // the next batch's raw values are fetched into registers while this batch is computed
  uint4 rq = make_uint4(0, 0, 0, 0), rk = rq, rv = rq;
  const int q8 = dim / 8, v8n = VW / 8;
  auto fetch = [&](int tb) {
    const int nt = min(kTB, t1 - tb);
    const int tq_ = tid / q8, dq = tid - tq_ * q8;
    if (tq_ < nt) {
      const T* row = proj + (size_t)(tb + tq_) * ld + (size_t)h * dim + dq * 8;
      if (OUT) rq = *reinterpret_cast<const uint4*>(row + q_off);
      rk = *reinterpret_cast<const uint4*>(row + k_off);
    }
    const int tv = tid / v8n, dv_ = tid - tv * v8n;
    rv = make_uint4(0, 0, 0, 0);
    if (tv < nt && v0 + dv_ * 8 < vdim)
      rv = *reinterpret_cast<const uint4*>(proj + (size_t)(tb + tv) * ld + v_off + (size_t)h * vdim + v0 + dv_ * 8);
  };
  auto stash = [&](int nt) {
    const int tq_ = tid / q8, dq = tid - tq_ * q8;
    if (tq_ < nt) {
      const __nv_bfloat16* bq = reinterpret_cast<const __nv_bfloat16*>(&rq);
      const __nv_bfloat16* bk = reinterpret_cast<const __nv_bfloat16*>(&rk);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (OUT) q_s[tq_ * dim + dq * 8 + e] = silu_f(__bfloat162float(bq[e]));
        k_s[tq_ * dim + dq * 8 + e] = silu_f(__bfloat162float(bk[e]));
      }
    }
    const int tv = tid / v8n, dv_ = tid - tv * v8n;
    if (tv < nt) {
      const __nv_bfloat16* bv = reinterpret_cast<const __nv_bfloat16*>(&rv);
#pragma unroll
      for (int e = 0; e < 8; ++e) v_s[tv * VW + dv_ * 8 + e] = silu_f(__bfloat162float(bv[e]));
    }
  };
  if (FAST && t0 < t1) fetch(t0);
  for (int tb = t0; tb < t1; tb += kTB) {
    const int nt = min(kTB, t1 - tb);
    __syncthreads();
    if (FAST) {
      stash(nt);
      __syncthreads();
      if (tb + kTB < t1) fetch(tb + kTB);
    } else {
      for (int i = tid; i < nt * dim; i += nthreads) {
        const int tt = i / dim, d = i - tt * dim;
        const T* row = proj + (size_t)(tb + tt) * ld + (size_t)h * dim + d;
        if (OUT) q_s[tt * dim + d] = silu_f(to_float<T>(row[q_off]));
        k_s[tt * dim + d] = silu_f(to_float<T>(row[k_off]));
      }
      for (int i = tid; i < nt * VW; i += nthreads) {
        const int tt = i / VW, vv = i - tt * VW;
        v_s[i] = v0 + vv < vdim
                     ? silu_f(to_float<T>(proj[(size_t)(tb + tt) * ld + v_off + (size_t)h * vdim + v0 + vv]))
                     : 0.f;
      }
      __syncthreads();
    }
    for (int tt = 0; tt < nt; ++tt) {
      float vt[VPT], acc[VPT];
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        vt[j] = v_s[tt * VW + j * kVS + tx];
        acc[j] = 0.f;
      }
      const float* kk = k_s + tt * dim + d0;
      const float* qq = q_s + tt * dim + d0;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        if (i < d_per && d0 + i < dim) {
          const float kv = kk[i];
#pragma unroll
          for (int j = 0; j < VPT; ++j) S[i][j] = fmaf(dec, S[i][j], kv * vt[j]);
          if (OUT) {
            const float qv = qq[i];
#pragma unroll
            for (int j = 0; j < VPT; ++j) acc[j] = fmaf(S[i][j], qv, acc[j]);
          }
        }
      }
      if (OUT) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) part[(ty * kTB + tt) * VW + j * kVS + tx] = acc[j];
      }
    }
    if (mode == 0) {
      __syncthreads();
      for (int i = tid; i < nt * VW; i += nthreads) {
        const int tt = i / VW, vv = i - tt * VW;
        if (v0 + vv < vdim) {
          float sum = 0.f;
          for (int p = 0; p < DP; ++p) sum += part[(p * kTB + tt) * VW + vv];
          out[(size_t)(tb + tt) * ldo + (size_t)h * vdim + v0 + vv] = sum;
        }
      }
    }
  }
  if (s_out != nullptr) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = d0 + i;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = v0 + j * kVS + tx;
        if (i < d_per && d < dim && v < vdim) s_out[(size_t)d * vdim + v] = S[i][j];
      }
    }
  }
}

// The pass over a sequence's chunks: entry c of chunk_state holds chunk c's own contribution D_c
// on entry and the state at chunk c's start on exit (for chunk 0 a copy of the slot's state, which
// the last chunk overwrites while the first may still read).  One thread per state element walks
// the chunks in order.
__global__ void linear_attention_chunk_prefix_kernel(float* chunk_state, const float* __restrict__ state,
                                                     const int* __restrict__ q_start,
                                                     const int* __restrict__ slot_ids,
                                                     const float* __restrict__ decay, int heads, int dim,
                                                     int vdim, int chunk, int n_seqs, int n_slots) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  const int s = blockIdx.y;
  const size_t per_seq = (size_t)heads * dim * vdim;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_seq) return;
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) return;
  int first = 0;
  for (int b = 0; b < s; ++b) first += (q_start[b + 1] - q_start[b] + chunk - 1) / chunk;
  const int nc = (q_start[s + 1] - q_start[s] + chunk - 1) / chunk;
  const int h = (int)(e / ((size_t)dim * vdim));
  float factor = 1.f;
  const float dec = decay[h];
  for (int i = 0; i < chunk; ++i) factor *= dec;       // decay^chunk, as chunk multiplications
  float run = state[(size_t)slot * per_seq + e];
  float carry = 0.f;       // D of the chunk before
  for (int c = 0; c < nc; ++c) {
    float* at = chunk_state + (size_t)(first + c) * per_seq + e;
    const float own = c + 1 < nc ? *at : 0.f;
    if (c > 0) run = fmaf(factor, run, carry);
    *at = run;
    carry = own;
  }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(256)
gate_norm_kernel(const float* __restrict__ o, int width, const TW* __restrict__ w, const T* __restrict__ gate,
                 int ldg, T* __restrict__ out, float eps) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float g = sigmoid_f(to_float<T>(gate[(size_t)t * ldg + c]));
    out[(size_t)t * width + c] = from_float<T>(row[c] * r * to_float<TW>(w[c]) * g);
  }
}

}  // namespace leone

using namespace leone;

// `proj`: [n_tokens, ld] in the run dtype with q, k (heads*dim each) and v (heads*vdim) at the given
// column offsets.  `out`: fp32 [n_tokens, ldo], head h at columns h*vdim.  `state`: fp32
// [n_slots, heads, dim, vdim].  chunk == 0: the walk in order; chunk > 0: the chunk-parallel form
// with `n_chunks` = sum over sequences of ceil(len / chunk) and `chunk_state` fp32
// [n_chunks, heads, dim, vdim].
extern "C" int leone_linear_attention(int dtype, const void* proj, int ld, int q_off, int k_off, int v_off,
                                      float* out, int ldo, float* state, const int* q_start,
                                      const int* slot_ids, const float* decay, int n_seqs, int heads,
                                      int dim, int vdim, int n_slots, int chunk, int n_chunks,
                                      float* chunk_state, int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || heads > 65535 || n_seqs > 65535 || dim > 512) return kRefusedSize;
  if (chunk < 0 || (chunk > 0 && (n_chunks <= 0 || n_chunks > 65535 || chunk_state == nullptr))) return kRefusedSize;
  // DP parts of the key dimension of at most 16 rows each (up to 8 parts), 1 or 4 value columns a thread
  int dp = (dim + 15) / 16;
  if (dp > 8) dp = 8;
  const int d_per = (dim + dp - 1) / dp;
  const int dpt = d_per <= 8 ? 8 : d_per <= 16 ? 16 : d_per <= 32 ? 32 : 64;
  const int vpt = (vdim > 32 && dpt <= 32) ? 4 : 1;
  const dim3 block(kVS, dp);
  const int vw = kVS * vpt;
  const size_t smem = sizeof(float) * ((size_t)2 * kTB * dim + kTB * vw + (size_t)dp * kTB * vw);
  const int vslices = (vdim + vw - 1) / vw;
  if (smem > 200 * 1024) return kRefusedSize;
  // the prefetching form: bfloat16, rows and offsets 16-byte aligned, one piece a thread and batch
  const int nthreads = kVS * dp;
  const bool fast = dtype == 1 && dim % 8 == 0 && vdim % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 &&
                    v_off % 8 == 0 && ((uintptr_t)proj % 16) == 0 && kTB * (dim / 8) <= nthreads &&
                    kTB * (vw / 8) <= nthreads;
#define SCAN(T, D, V, GRIDZ, OUT, FAST)                                                                    \
  do {                                                                                                     \
    auto kern = linear_attention_scan_kernel<T, D, V, OUT, FAST>;                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_kernel(kern, dim3(vslices, heads, GRIDZ), block, smem, stream,                                             \
        (const T*)proj, ld, q_off, k_off, v_off, out, ldo, state, chunk_state, q_start, slot_ids, decay,   \
        heads, dim, vdim, chunk, n_seqs, n_slots, status);                                                 \
  } while (0)
#define SCAN_F(T, D, V, GRIDZ, OUT)                                     \
  do {                                                                  \
    if (fast && sizeof(T) == 2) SCAN(T, D, V, GRIDZ, OUT, true);        \
    else SCAN(T, D, V, GRIDZ, OUT, false);                              \
  } while (0)
#define SCAN_D(T, GRIDZ, OUT)                                       \
  do {                                                              \
    if (vpt == 4) {                                                 \
      if (dpt == 8) SCAN_F(T, 8, 4, GRIDZ, OUT);                    \
      else if (dpt == 16) SCAN_F(T, 16, 4, GRIDZ, OUT);             \
      else SCAN_F(T, 32, 4, GRIDZ, OUT);                            \
    } else {                                                        \
      if (dpt == 8) SCAN_F(T, 8, 1, GRIDZ, OUT);                    \
      else if (dpt == 16) SCAN_F(T, 16, 1, GRIDZ, OUT);             \
      else if (dpt == 32) SCAN_F(T, 32, 1, GRIDZ, OUT);             \
      else SCAN_F(T, 64, 1, GRIDZ, OUT);                            \
    }                                                               \
  } while (0)
#define SCAN_T(GRIDZ, OUT)                              \
  do {                                                  \
    if (dtype == 0) SCAN_D(float, GRIDZ, OUT);          \
    else SCAN_D(__nv_bfloat16, GRIDZ, OUT);             \
  } while (0)
  if (dtype != 0 && dtype != 1) return kRefusedDtype;
  if (chunk == 0) {
    SCAN_T(n_seqs, true);
    return launch_result();
  }
  SCAN_T(n_chunks, false);
  const size_t per_seq = (size_t)heads * dim * vdim;
  launch_kernel(linear_attention_chunk_prefix_kernel, dim3((unsigned)((per_seq + 255) / 256), n_seqs), dim3(256), 0, stream, 
      chunk_state, state, q_start, slot_ids, decay, heads, dim, vdim, chunk, n_seqs, n_slots);
  SCAN_T(n_chunks, true);
#undef SCAN_T
#undef SCAN_F
#undef SCAN_D
#undef SCAN
  return launch_result();
}

// out[t, c] = o[t, c] / sqrt(mean_c(o[t, :]^2) + eps) * w[c] * sigmoid(gate[t, c]); o fp32, out and
// gate in the run dtype (gate rows `ldg` apart), w in `w_dtype`.
extern "C" int leone_gate_norm(int dtype, const float* o, int n_tokens, int width, const void* w, int w_dtype,
                               const void* gate, int ldg, void* out, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (width <= 0) return kRefusedSize;
#define GN(T, TW) \
  launch_kernel(gate_norm_kernel<T, TW>, dim3(n_tokens), dim3(256), 0, stream, o, width, (const TW*)w, (const T*)gate, ldg, (T*)out, eps)
  if (dtype == 0 && w_dtype == 0) GN(float, float);
  else if (dtype == 1 && w_dtype == 0) GN(__nv_bfloat16, float);
  else if (dtype == 1 && w_dtype == 1) GN(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == 0 && w_dtype == 1) GN(float, __nv_bfloat16);
  else return kRefusedDtype;
#undef GN
  return launch_result();
}
