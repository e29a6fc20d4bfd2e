// What lies between the input projection of an attention and its score kernel, and behind the score kernel, for
// attentions without the rotate-half form: biases, norms per head, a position-dependent stretch of the query, the
// latent form of keys and values, and output gates.  All statistics, angles and factors are 32-bit.
//
// qk_norm_kv_write: rows of the projection are [nq query heads | nkv key heads] of kd values, then nkv value heads of
//   vd values.  Optional biases are added; query and key heads are divided by sqrt(mean(x^2) + eps) and multiplied by
//   a weight of kd values shared by the heads (no weights: no norm); the query is further multiplied by
//   1 + coef * ln(floor((p + 1) / every) + 1) at position p (every = 0: not).  With a frequency table the first
//   rot_dims values of every query and key head are then turned by p * freq[i], value i with i + rot_dims / 2 or value
//   2i with 2i + 1, cos and sin times a constant.  Queries are rewritten in place, keys and values go to their pages.
//   One warp per head row.
// latent_kv_write: rows are [nq query heads of (nd plain | rd rotated) values | rank latent values | rd rotated key
//   values | ...].  The latent is normed (weight of rank values) and written both as the first `rank` values of the
//   token's key row and as its value row; the key's rotated part and every query head's rotated part are turned in
//   pairs (2i, 2i + 1), i < rot_dims / 2, by p * freq[i]; the key part goes behind the latent in the key row, the
//   query parts to q_out[t, head, rank : rank + rd].  (The plain query parts reach q_out through a product with the
//   keys' up-projection, which is not this kernel's.)
// sigmoid_gate: out[t, h, :] = x[t, h, :] * sigmoid(gate), the gate one value per element or one per head.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int MAX_ROW = 512;   // values of a head row or of the latent

struct QkArgs {
  void* proj;
  int ld, nq, nkv, kd, vd;
  const float *bq, *bk, *bv;    // biases [nq * kd], [nkv * kd], [nkv * vd] or null
  const float *wq, *wk;         // norm weights [kd] or null
  float eps, coef;
  int every;
  const int* positions;
  void *kcache, *vcache;
  const int* slot_mapping;
  int page_size;
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
  int n_tokens;
  const float* freq;            // [rot_dims / 2] or null: query and key heads are rotated behind the norm
  int rot_dims, rot_pairs;      // the first rot_dims values of a head turn; pairs (2i, 2i + 1) or halves (i, i + rot_dims / 2)
  float rot_mag;                // cos and sin are multiplied by this
};

template <typename T>
__global__ void __launch_bounds__(128) qk_norm_kv_write_kernel(QkArgs a) {
  __shared__ float turned[4][MAX_ROW];
  pdl_trigger();
  pdl_wait();
  const int rows = a.nq + 2 * a.nkv;
  const long long task = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (task >= (long long)a.n_tokens * rows) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(task / rows), r = (int)(task % rows);
  T* row = (T*)a.proj + (size_t)t * a.ld;
  const int slot = a.slot_mapping[t];
  const long long page = slot / a.page_size, off = slot % a.page_size;
  if (r >= a.nq + a.nkv) {   // a value head: bias, then to its page
    if (slot < 0) return;
    const int h = r - a.nq - a.nkv;
    const T* src = row + (size_t)(a.nq + a.nkv) * a.kd + (size_t)h * a.vd;
    T* dst = (T*)a.vcache + page * a.v_page_stride + (long long)h * a.v_head_stride + off * a.vd;
    for (int d = lane; d < a.vd; d += 32)
      dst[d] = from_f32<T>(to_f32(src[d]) + (a.bv ? a.bv[h * a.vd + d] : 0.f));
    return;
  }
  const bool is_q = r < a.nq;
  if (!is_q && slot < 0) return;
  const int h = is_q ? r : r - a.nq;
  const float* bias = is_q ? a.bq : a.bk;
  const float* w = is_q ? a.wq : a.wk;
  T* src = row + (size_t)r * a.kd;
  float x[MAX_ROW / 32];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_ROW / 32; ++i) {
    const int d = lane + 32 * i;
    x[i] = d < a.kd ? to_f32(src[d]) + (bias ? bias[h * a.kd + d] : 0.f) : 0.f;
    ss = fmaf(x[i], x[i], ss);
  }
  float f = 1.f;
  if (w) f = 1.f / sqrtf(warp_sum(ss) / (float)a.kd + a.eps);
  float stretch = 1.f;
  if (is_q && a.every > 0) stretch = fmaf(a.coef, logf((float)((a.positions[t] + 1) / a.every + 1)), 1.f);
  T* dst = is_q ? src : (T*)a.kcache + page * a.k_page_stride + (long long)h * a.k_head_stride + off * a.kd;
  float* mine = turned[threadIdx.x >> 5];
#pragma unroll
  for (int i = 0; i < MAX_ROW / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < a.kd) {
      float y = w ? __fmul_rn(__fmul_rn(x[i], f), w[d]) : x[i];
      if (is_q) y = __fmul_rn(y, stretch);
      if (a.rot_dims > 0) mine[d] = y;
      else dst[d] = from_f32<T>(y);
    }
  }
  if (a.rot_dims == 0) return;
  // the rotation reads the normed values in 32-bit (the partner of a value lies with another lane) and rounds once
  __syncwarp();
  const float pos = (float)a.positions[t];
  const int half = a.rot_dims / 2;
  for (int d = lane; d < a.kd; d += 32) {
    float y = mine[d];
    if (d < a.rot_dims) {
      const int i = a.rot_pairs ? d >> 1 : (d < half ? d : d - half);
      const bool first = a.rot_pairs ? !(d & 1) : d < half;
      const float u = mine[a.rot_pairs ? 2 * i : i], v = mine[a.rot_pairs ? 2 * i + 1 : i + half];
      const float ang = __fmul_rn(pos, a.freq[i]);
      const float c = __fmul_rn(cosf(ang), a.rot_mag), sn = __fmul_rn(sinf(ang), a.rot_mag);
      y = first ? fmaf(u, c, -__fmul_rn(v, sn)) : fmaf(v, c, __fmul_rn(u, sn));
    }
    dst[d] = from_f32<T>(y);
  }
}

struct LatentArgs {
  const void* proj;
  int ld, nq, nd, rd, rank, rot_dims;
  const float* w_latent;     // [rank]
  const float* freq;         // [rot_dims / 2]
  float eps;
  const int* positions;
  void* q_out;               // [T, nq, rank + rd]
  void *kcache, *vcache;     // key rows of rank + rd values, value rows of rank values, one head
  const int* slot_mapping;
  int page_size;
  long long k_page_stride, v_page_stride;
  int n_tokens;
  float rot_mag;             // cos and sin are multiplied by this
};

// With kcache == null the rows hold queries only: their rotated parts are turned and nothing is written to a cache
// (a mixer that reads the latents and key parts another layer cached).
// One CTA of 128 threads per token: warp 0 norms the latent, all threads turn the rotated parts.
template <typename T>
__global__ void __launch_bounds__(128) latent_kv_write_kernel(LatentArgs a) {
  __shared__ float cs[256], sn[256];   // rot_dims / 2 <= 256
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= a.n_tokens) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float pos = (float)a.positions[t];
  for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
    const float ang = __fmul_rn(pos, a.freq[i]);
    cs[i] = __fmul_rn(cosf(ang), a.rot_mag);
    sn[i] = __fmul_rn(sinf(ang), a.rot_mag);
  }
  __syncthreads();
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  const int qd = a.nd + a.rd, kd = a.rank + a.rd;
  const T* lat = row + (size_t)a.nq * qd;
  const bool writes = a.kcache != nullptr;
  const int slot = writes ? a.slot_mapping[t] : -1;
  const long long page = slot / a.page_size, off = slot % a.page_size;
  T* krow = (T*)a.kcache + page * a.k_page_stride + off * kd;
  T* vrow = (T*)a.vcache + page * a.v_page_stride + off * a.rank;
  if (warp == 0 && slot >= 0) {
    float x[MAX_ROW / 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_ROW / 32; ++i) {
      const int d = lane + 32 * i;
      x[i] = d < a.rank ? to_f32(lat[d]) : 0.f;
      ss = fmaf(x[i], x[i], ss);
    }
    const float f = 1.f / sqrtf(warp_sum(ss) / (float)a.rank + a.eps);
#pragma unroll
    for (int i = 0; i < MAX_ROW / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < a.rank) {
        const T y = from_f32<T>(__fmul_rn(__fmul_rn(x[i], f), a.w_latent[d]));
        krow[d] = y;
        vrow[d] = y;
      }
    }
  }
  // rotated parts: unit 0 is the key's, unit 1 + h query head h's; pairs (2i, 2i + 1)
  const int half = (a.rd + 1) / 2, half_rot = a.rot_dims / 2;
  for (int idx = threadIdx.x; idx < (a.nq + 1) * half; idx += blockDim.x) {
    const int u = idx / half, i = idx % half;
    if (u == 0 && slot < 0) continue;
    const T* src = (u == 0 ? lat + a.rank : row + (size_t)(u - 1) * qd + a.nd) + 2 * i;
    T* dst = (u == 0 ? krow + a.rank : (T*)a.q_out + ((size_t)t * a.nq + (u - 1)) * kd + a.rank) + 2 * i;
    const bool pair = 2 * i + 1 < a.rd;
    const float x = to_f32(src[0]), y = pair ? to_f32(src[1]) : 0.f;
    float ox = x, oy = y;
    if (i < half_rot) {
      const float c = cs[i], s = sn[i];
      ox = fmaf(x, c, -__fmul_rn(y, s));
      oy = fmaf(y, c, __fmul_rn(x, s));
    }
    dst[0] = from_f32<T>(ox);
    if (pair) dst[1] = from_f32<T>(oy);
  }
}

// x float32 [T, heads * vd]; gate rows of ldg values in the engine's dtype, heads * vd of them (per_head = 0) or
// `heads` (per_head = 1); out [T, heads * vd] in the engine's dtype.
template <typename T>
__global__ void sigmoid_gate_kernel(const float* __restrict__ x, const T* __restrict__ gate, int ldg, int per_head,
                                    T* __restrict__ out, long long n_tokens, int heads, int vd) {
  pdl_trigger();
  pdl_wait();
  const long long width = (long long)heads * vd, total = n_tokens * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width;
    const int c = (int)(idx % width);
    const float g = to_f32(gate[t * ldg + (per_head ? c / vd : c)]);
    out[idx] = from_f32<T>(x[idx] / (1.f + expf(-g)));
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_qk_norm_kv_write(void* proj, int ld, int nq, int nkv, int kd, int vd, const float* bq, const float* bk,
                                     const float* bv, const float* wq, const float* wk, float eps, float coef, int every,
                                     const int* positions, void* kcache, void* vcache, const int* slot_mapping,
                                     int page_size, long long k_page_stride, long long k_head_stride,
                                     long long v_page_stride, long long v_head_stride, int n_tokens, const float* freq,
                                     int rot_dims, int rot_pairs, float rot_mag, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && kd > 0 && kd <= MAX_ROW && vd > 0,
               "qk_norm_kv_write: %d tokens, %d / %d heads, key size %d (at most %d), value size %d", n_tokens, nq, nkv, kd, MAX_ROW, vd);
  TLLM_REQUIRE((wq == nullptr) == (wk == nullptr) && every >= 0 && page_size > 0 && kcache && vcache && slot_mapping && positions,
               "qk_norm_kv_write: norm weights for both of queries and keys or neither; caches, slots and positions are needed");
  QkArgs a;
  a.proj = proj; a.ld = ld; a.nq = nq; a.nkv = nkv; a.kd = kd; a.vd = vd; a.bq = bq; a.bk = bk; a.bv = bv; a.wq = wq; a.wk = wk;
  a.eps = eps; a.coef = coef; a.every = every; a.positions = positions; a.kcache = kcache; a.vcache = vcache;
  a.slot_mapping = slot_mapping; a.page_size = page_size; a.k_page_stride = k_page_stride; a.k_head_stride = k_head_stride;
  a.v_page_stride = v_page_stride; a.v_head_stride = v_head_stride; a.n_tokens = n_tokens;
  TLLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= kd && (rot_dims == 0 || freq),
               "qk_norm_kv_write: %d rotated values of %d (even, at most the head's size, with a frequency table)", rot_dims, kd);
  a.freq = freq; a.rot_dims = rot_dims; a.rot_pairs = rot_pairs; a.rot_mag = rot_mag;
  const long long tasks = (long long)n_tokens * (nq + 2 * nkv), blocks = (tasks + 3) / 4;
  TLLM_REQUIRE(blocks <= 2147483647LL, "qk_norm_kv_write: %lld rows exceed the grid", tasks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32) TLLM_LAUNCH("qk_norm_kv_write", qk_norm_kv_write_kernel<float>, (unsigned)blocks, 128, 0, s, a);
  else if (dtype == TLLM_BF16) TLLM_LAUNCH("qk_norm_kv_write", qk_norm_kv_write_kernel<__nv_bfloat16>, (unsigned)blocks, 128, 0, s, a);
  else TLLM_FAIL(TLLM_ERR_ARG, "qk_norm_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_latent_kv_write(const void* proj, int ld, int nq, int nd, int rd, int rank, int rot_dims,
                                    const float* w_latent, const float* freq, float eps, const int* positions, void* q_out,
                                    void* kcache, void* vcache, const int* slot_mapping, int page_size,
                                    long long k_page_stride, long long v_page_stride, int n_tokens, float rot_mag,
                                    int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nd >= 0 && rd >= 0 && rank > 0 && rank <= MAX_ROW,
               "latent_kv_write: %d tokens, %d heads, sizes %d + %d, latent %d (at most %d)", n_tokens, nq, nd, rd, rank, MAX_ROW);
  TLLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rd && rot_dims <= 512 && (rot_dims == 0 || freq),
               "latent_kv_write: %d rotated values of %d (even, at most the part's size and 512, with a frequency table)", rot_dims, rd);
  TLLM_REQUIRE(positions && q_out && page_size > 0 && (kcache == nullptr || (w_latent && vcache && slot_mapping)), "latent_kv_write: a pointer is missing");
  LatentArgs a;
  a.proj = proj; a.ld = ld; a.nq = nq; a.nd = nd; a.rd = rd; a.rank = rank; a.rot_dims = rot_dims; a.w_latent = w_latent;
  a.freq = freq; a.eps = eps; a.positions = positions; a.q_out = q_out; a.kcache = kcache; a.vcache = vcache;
  a.slot_mapping = slot_mapping; a.page_size = page_size; a.k_page_stride = k_page_stride; a.v_page_stride = v_page_stride;
  a.n_tokens = n_tokens; a.rot_mag = rot_mag;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32) TLLM_LAUNCH("latent_kv_write", latent_kv_write_kernel<float>, n_tokens, 128, 0, s, a);
  else if (dtype == TLLM_BF16) TLLM_LAUNCH("latent_kv_write", latent_kv_write_kernel<__nv_bfloat16>, n_tokens, 128, 0, s, a);
  else TLLM_FAIL(TLLM_ERR_ARG, "latent_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_sigmoid_gate(const float* x, const void* gate, int ldg, int per_head, void* out, long long n_tokens,
                                 int heads, int vd, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && heads > 0 && vd > 0, "sigmoid_gate: %lld tokens, %d heads of %d values", n_tokens, heads, vd);
  const long long total = n_tokens * heads * vd;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("sigmoid_gate", sigmoid_gate_kernel<float>, blocks, threads, 0, s, x, (const float*)gate, ldg, per_head, (float*)out, n_tokens, heads, vd);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("sigmoid_gate", sigmoid_gate_kernel<__nv_bfloat16>, blocks, threads, 0, s, x, (const __nv_bfloat16*)gate, ldg, per_head, (__nv_bfloat16*)out, n_tokens, heads, vd);
  else TLLM_FAIL(TLLM_ERR_ARG, "sigmoid_gate: unknown dtype code %d", dtype);
  return TLLM_OK;
}
