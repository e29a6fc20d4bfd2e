// Memory-bound kernels of the step: embedding gather, RMSNorm, SiLU*up, and the fused
// rotate-and-cache kernel (RoPE on queries and keys in 32-bit, keys and values written into
// their pages).  All take float32 or bfloat16 activations; statistics and angles are 32-bit.
// Reference counterparts: tiny_llm/ops/cuda/embedding.cu:10-29, norm.cu:16-49, silu.cu:7-12,
// arithmetic.cu:7-22, rope.cu:26-95, gemm.cu:380-411 (the scatter of K/V rows into pages).
#include <algorithm>
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

// ---------------------------------------------------------------- embedding: out[t,:] = table[tokens[t],:] * scale
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int n_tokens, int hidden, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const T* row = table + (size_t)tokens[t] * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = __fmul_rn(to_f32(row[i]), scale);
}

// ---------------------------------------------------------------- RMSNorm
// y_j = (w_j * x_j) / sqrt(sum_j(x_j^2)/H + eps); one block per row; rows may be gathered.
template <typename T>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                T* __restrict__ out, const int* __restrict__ rows, int n_rows,
                                int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = src[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);   // one division per row; the elements are multiplied
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>((w[i] * src[i]) * inv);
}

// resid_j += scale * w_j * x_j / sqrt(sum_j(x_j^2)/H + eps): a branch that is normed before it joins the stream.
// clear != 0: x is handed back zeroed (a branch buffer that products accumulate into).
__global__ void rms_norm_add_kernel(float* __restrict__ x, const float* __restrict__ w, float* __restrict__ resid,
                                    int n_rows, int hidden, float eps, float scale, int clear,
                                    __nv_bfloat16* __restrict__ copy) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  float* src = x + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = src[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);
  float* dst = resid + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float y = dst[i] + scale * ((w[i] * src[i]) * inv);
    dst[i] = y;
    if (copy) copy[(size_t)r * hidden + i] = __float2bfloat16_rn(y);   // the stream as the next branch reads it
    if (clear) src[i] = 0.f;
  }
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  uint2 pk;
  *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = pk;
}

// The same for widths that are multiples of 4 and at most 4 * VEC * blockDim: the row is read once,
// with 16-byte loads, and kept in registers between the two passes.
template <typename T, int VEC>
__global__ void rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    T* __restrict__ out, const int* __restrict__ rows, int n_rows,
                                    int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  // the weight is a constant of the model (and `rows` comes with the step's tables): both are read
  // before the wait for the kernel that writes x, so that only x itself is waited for afterwards
  const int r = blockIdx.x;
  const int n4 = hidden / 4;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 g[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    g[i] = idx < n4 ? __ldg(w4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src_row = r < n_rows ? (rows ? rows[r] : r) : 0;
  pdl_wait();
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)src_row * hidden);
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    v[i] = idx < n4 ? src[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);   // one division per row; the elements are multiplied
  T* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4)
      store4(dst + 4 * idx, (g[i].x * v[i].x) * inv, (g[i].y * v[i].y) * inv, (g[i].z * v[i].z) * inv, (g[i].w * v[i].w) * inv);
  }
}

// ---------------------------------------------------------------- act(gate) * up, act = SiLU (0) or ReLU (1)
// `gu` rows hold gate and up interleaved in blocks: [2 g B, 2 g B + B) gate, next B up.  With
// ZERO the source is a float32 accumulation buffer (split-K partial sums land there) that this
// kernel hands back cleared: every element is read once, by the thread that then zeroes it.
template <typename TIn, typename TOut, bool ZERO>
__global__ void silu_mul_kernel(TIn* __restrict__ gu, TOut* __restrict__ out, int m, int inter, int blk, int act) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)m * inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(idx / inter), col = (int)(idx % inter);
    const int g = col / blk, j = col % blk;
    TIn* src = gu + (size_t)row * 2 * inter + (size_t)g * 2 * blk;
    const float gate = to_f32(src[j]), up = to_f32(src[blk + j]);
    if (ZERO) { src[j] = from_f32<TIn>(0.f); src[blk + j] = from_f32<TIn>(0.f); }
    out[idx] = from_f32<TOut>((act == 1 ? fmaxf(gate, 0.f) : gate / (1.f + expf(-gate))) * up);
  }
}

// The same from float32 sums, four neighbouring outputs per thread (the block and the row are multiples of four values
// and the rows 16-byte aligned): two 16-byte loads, one store.  ZERO hands the sums back cleared.
template <typename TOut, bool ZERO>
__global__ void __launch_bounds__(256) silu_mul_f32x4_kernel(float* __restrict__ gu, TOut* __restrict__ out, int m, int inter,
                                                             int blk, int act) {
  pdl_trigger();
  pdl_wait();
  const int per_row = inter >> 2;
  const long long total = (long long)m * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx / per_row), col = (int)(idx - (long long)row * per_row) << 2;
    const int g = col / blk, j = col - g * blk;
    float* src = gu + (size_t)row * 2 * inter + (size_t)g * 2 * blk + j;
    const float4 gate = *reinterpret_cast<const float4*>(src), up = *reinterpret_cast<const float4*>(src + blk);
    if (ZERO) {
      *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(src + blk) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float gv[4] = {gate.x, gate.y, gate.z, gate.w}, uv[4] = {up.x, up.y, up.z, up.w};
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = (act == 1 ? fmaxf(gv[i], 0.f) : gv[i] / (1.f + expf(-gv[i]))) * uv[i];
    TOut* dst = out + (size_t)row * inter + col;
    if constexpr (sizeof(TOut) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(dst) = pk;
    } else {
      *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
    }
  }
}

// ---------------------------------------------------------------- rotate and cache
// qkv row: [nq*hd queries | nkv*hd keys | nkv*hd values] (keys/values absent when slot_mapping is
// null).  Queries are rotated in place; keys are rotated and written to the key pages, values are
// copied to the value pages, both at slot_mapping[t] = page*page_size + offset.
// Rotation (rotate-half over the whole head; rot_dim is hd or 0): x'_i = c x_i - s x_{i+hd/2},
// x'_{i+hd/2} = s x_i + c x_{i+hd/2}.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, float* __restrict__ src, int src_stride,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     int n_tokens, int nq, int nkv, int hd, int row_stride,
                                     T* __restrict__ kcache, T* __restrict__ vcache,
                                     const int* __restrict__ slot_mapping, int page_size,
                                     long long page_stride, long long head_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride;
  float* srow = src ? src + (size_t)t * src_stride : nullptr;   // float32 source that is handed back zeroed
  const bool write_kv = slot_mapping != nullptr;
  const int heads = write_kv ? nq + nkv : nq;
  const int half_hd = hd / 2;
  long long slot_base = 0;
  if (write_kv) {
    const int slot = slot_mapping[t];
    if (slot < 0) return;   // a token without a slot writes nothing
    slot_base = (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * hd;
  }
  // queries and keys: one thread per (head, i < hd/2) rotates the pair of dims (i, i + hd/2)
  for (int idx = threadIdx.x; idx < heads * half_hd; idx += blockDim.x) {
    const int h = idx / half_hd, i = idx % half_hd;
    const int e = h * hd + i;
    float va, vb;
    if (srow) {
      // the projection's output is a tensor of the model's dtype: its sums are rounded to it before the rotation,
      // as where the projection itself stores them
      va = to_f32(from_f32<T>(srow[e])); vb = to_f32(from_f32<T>(srow[e + half_hd]));
      srow[e] = 0.f; srow[e + half_hd] = 0.f;
    } else {
      va = to_f32(row[e]); vb = to_f32(row[e + half_hd]);
    }
    float oa = va, ob = vb;
    if (cos_t) {
      const float c = cos_t[(size_t)pos * half_hd + i], s = sin_t[(size_t)pos * half_hd + i];
      oa = c * va - s * vb;
      ob = s * va + c * vb;
    }
    T* dst = h < nq ? row + (size_t)h * hd : kcache + slot_base + (long long)(h - nq) * head_stride;
    dst[i] = from_f32<T>(oa);
    dst[i + half_hd] = from_f32<T>(ob);
  }
  if (write_kv) {
    const int v0 = (nq + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
      const int h = idx / hd, i = idx % hd;
      T val;
      if (srow) { val = from_f32<T>(srow[v0 + idx]); srow[v0 + idx] = 0.f; }
      else val = row[v0 + idx];
      vcache[slot_base + (long long)h * head_stride + i] = val;
    }
  }
}

// ---- the same with 16-byte accesses, for head sizes that are multiples of 16 and aligned rows:
// one thread rotates eight consecutive pairs (i, i + hd/2).
__device__ __forceinline__ void load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, float* __restrict__ src, int src_stride,
                                         const int* __restrict__ positions,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         int n_tokens, int nq, int nkv, int hd, int row_stride,
                                         T* __restrict__ kcache, T* __restrict__ vcache,
                                         const int* __restrict__ slot_mapping, int page_size,
                                         long long page_stride, long long head_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride;
  float* srow = src ? src + (size_t)t * src_stride : nullptr;
  const bool write_kv = slot_mapping != nullptr;
  const int heads = write_kv ? nq + nkv : nq;
  const int half_hd = hd / 2, groups = half_hd / 8;   // groups of eight pairs per head
  long long slot_base = 0;
  if (write_kv) {
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    slot_base = (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * hd;
  }
  const float zeros[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  // gridDim.y CTAs share a token's work items
  const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
  for (int idx = first; idx < heads * groups; idx += step) {
    const int h = idx / groups, i = (idx % groups) * 8;
    const int e = h * hd + i;
    float va[8], vb[8], oa[8], ob[8];
    if (srow) {
      load8(srow + e, va); load8(srow + e + half_hd, vb);
      store8(srow + e, zeros); store8(srow + e + half_hd, zeros);
#pragma unroll
      for (int j = 0; j < 8; ++j) { va[j] = to_f32(from_f32<T>(va[j])); vb[j] = to_f32(from_f32<T>(vb[j])); }   // (as above)
    } else {
      load8(row + e, va); load8(row + e + half_hd, vb);
    }
    if (cos_t) {
      float c[8], sn[8];
      load8(cos_t + (size_t)pos * half_hd + i, c);
      load8(sin_t + (size_t)pos * half_hd + i, sn);
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = c[j] * va[j] - sn[j] * vb[j]; ob[j] = sn[j] * va[j] + c[j] * vb[j]; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = va[j]; ob[j] = vb[j]; }
    }
    T* dst = h < nq ? row + (size_t)h * hd : kcache + slot_base + (long long)(h - nq) * head_stride;
    store8(dst + i, oa);
    store8(dst + i + half_hd, ob);
  }
  if (write_kv) {
    const int v0 = (nq + nkv) * hd;
    for (int idx = first; idx < nkv * hd / 8; idx += step) {
      const int h = (idx * 8) / hd, i = (idx * 8) % hd;
      float v[8];
      if (srow) { load8(srow + v0 + idx * 8, v); store8(srow + v0 + idx * 8, zeros); }
      else load8(row + v0 + idx * 8, v);
      store8(vcache + slot_base + (long long)h * head_stride + i, v);
    }
  }
}


// ---------------------------------------------------------------- embedding added into the stream: out[t,:] += table[tokens[t],:]
// (a model that runs a span of layers several times adds the embedding output again before each further pass)
template <typename T>
__global__ void embedding_add_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                     float* __restrict__ out, int n_tokens, int hidden) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const T* row = table + (size_t)tokens[t] * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] += to_f32(row[i]);
}

// ---------------------------------------------------------------- Dynamic Tanh
// y_j = tanh(alpha x_j) w_j + b_j: a norm without statistics; alpha is one number of the model, read from the device.
template <typename T>
__global__ void dyt_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                const float* __restrict__ alpha, T* __restrict__ out, const int* __restrict__ rows,
                                int n_rows, int hidden) {
  pdl_trigger();
  const float a = __ldg(alpha);
  const int r = blockIdx.x;
  const int src_row = r < n_rows ? (rows ? rows[r] : r) : 0;
  pdl_wait();
  if (r >= n_rows) return;
  const float* src = x + (size_t)src_row * hidden;
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>(fmaf(tanhf(a * src[i]), w[i], b[i]));
}

// The same with 16-byte accesses, for widths that are multiples of 4 and aligned rows; several rows per CTA when
// there are many, so that the weight and bias vectors are read once per CTA and not once per row.
template <typename T>
__global__ void dyt_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                    const float* __restrict__ alpha, T* __restrict__ out, const int* __restrict__ rows,
                                    int n_rows, int hidden, int rows_per_cta) {
  pdl_trigger();
  const float a = __ldg(alpha);
  const int n4 = hidden / 4;
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(n_rows, r0 + rows_per_cta);
  pdl_wait();
  for (int idx = threadIdx.x; idx < n4; idx += blockDim.x) {
    const float4 wv = __ldg(reinterpret_cast<const float4*>(w) + idx), bv = __ldg(reinterpret_cast<const float4*>(b) + idx);
    for (int r = r0; r < r1; ++r) {
      const float4 v = *(reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden) + idx);
      store4(out + (size_t)r * hidden + 4 * idx, fmaf(tanhf(a * v.x), wv.x, bv.x), fmaf(tanhf(a * v.y), wv.y, bv.y),
             fmaf(tanhf(a * v.z), wv.z, bv.z), fmaf(tanhf(a * v.w), wv.w, bv.w));
    }
  }
}

// ---------------------------------------------------------------- rotate pairs and cache
// qkv row: [nq*kd queries | nk*kd keys | nv*vd values]; nq and nk count rows of kd values (heads times score maps).
// The first rot_dims values of every query and key row are rotated, value 2i with value 2i+1, by the angle
// pos * freq[i] (angle, cosine and sine in 32-bit); the rest pass unchanged.  Queries are rewritten in place; keys go
// to the key pages (rows of kd values, nk per slot), values to the value pages (rows of vd values, nv per slot).
template <typename T>
__global__ void rope_pairs_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                           const float* __restrict__ freq, int rot_dims, int n_tokens, int nq, int nk,
                                           int nv, int kd, int vd, int row_stride, T* __restrict__ kcache,
                                           T* __restrict__ vcache, const int* __restrict__ slot_mapping, int page_size,
                                           long long k_page_stride, long long k_head_stride, long long v_page_stride,
                                           long long v_head_stride) {
  __shared__ float cs[256], sn[256];   // rot_dims / 2 <= 256
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const float pos = (float)positions[t];
  const int half_rot = rot_dims / 2, half_kd = (kd + 1) / 2;   // an odd key size ends in a value without a partner
  for (int i = threadIdx.x; i < half_rot; i += blockDim.x) {
    const float ang = __fmul_rn(pos, freq[i]);
    cs[i] = cosf(ang);
    sn[i] = sinf(ang);
  }
  __syncthreads();
  T* row = qkv + (size_t)t * row_stride;
  const int slot = slot_mapping[t];
  if (slot < 0) return;   // a token without a slot writes nothing
  const long long page = slot / page_size, off = slot % page_size;
  T* kbase = kcache + page * k_page_stride + off * kd;
  T* vbase = vcache + page * v_page_stride + off * vd;
  for (int idx = threadIdx.x; idx < (nq + nk) * half_kd; idx += blockDim.x) {
    const int h = idx / half_kd, i = idx % half_kd;
    const T* srcp = row + (size_t)h * kd + 2 * i;
    const bool pair = 2 * i + 1 < kd;
    const float u = to_f32(srcp[0]), v = pair ? to_f32(srcp[1]) : 0.f;
    float ou = u, ov = v;
    if (i < half_rot) {
      const float c = cs[i], s = sn[i];
      ou = fmaf(u, c, -__fmul_rn(v, s));
      ov = fmaf(v, c, __fmul_rn(u, s));
    }
    T* dst = h < nq ? row + (size_t)h * kd + 2 * i : kbase + (long long)(h - nq) * k_head_stride + 2 * i;
    dst[0] = from_f32<T>(ou);
    if (pair) dst[1] = from_f32<T>(ov);
  }
  const T* vsrc = row + (size_t)(nq + nk) * kd;
  for (int idx = threadIdx.x; idx < nv * vd; idx += blockDim.x) {
    const int h = idx / vd, i = idx % vd;
    vbase[(long long)h * v_head_stride + i] = vsrc[idx];
  }
}

// ---------------------------------------------------------------- differential combine
// a: float32 [T, heads, 2, vd], the outputs of a head's two score maps over the same values.
// lambda = exp(sum(lq1 lk1)) - exp(sum(lq2 lk2)) + diff (one number of the layer, recomputed by every warp in the same
// order); o = a1 - lambda a2; out = o / sqrt(mean(o^2) + eps) * (1 - diff).  One warp per (token, head); vd <= 256.
template <typename T>
__global__ void diff_combine_kernel(const float* __restrict__ a, const float* __restrict__ lq1, const float* __restrict__ lk1,
                                    const float* __restrict__ lq2, const float* __restrict__ lk2, int kd, float diff,
                                    float eps, T* __restrict__ out, long long n_rows, int vd) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < kd; i += 32) { s1 = fmaf(lq1[i], lk1[i], s1); s2 = fmaf(lq2[i], lk2[i], s2); }
  s1 = warp_sum(s1); s2 = warp_sum(s2);
  const float lambda = expf(s1) - expf(s2) + diff;
  pdl_wait();
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float* a1 = a + r * 2 * vd;
  const float* a2 = a1 + vd;
  float o[8];
  float ss = 0.f;
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int d = lane + 32 * x;
    o[x] = d < vd ? fmaf(-lambda, a2[d], a1[d]) : 0.f;
    ss = fmaf(o[x], o[x], ss);
  }
  ss = warp_sum(ss);
  const float inv = (1.f - diff) / sqrtf(ss / (float)vd + eps);
  T* dst = out + r * vd;
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int d = lane + 32 * x;
    if (d < vd) dst[d] = from_f32<T>(o[x] * inv);
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_embedding_add(const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                                  int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && hidden > 0, "embedding_add: empty input (%d tokens, width %d)", n_tokens, hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("embedding_add", embedding_add_kernel<float>, n_tokens, threads, 0, s, tokens, (const float*)table, out, n_tokens, hidden);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("embedding_add", embedding_add_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, tokens, (const __nv_bfloat16*)table, out, n_tokens, hidden);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "embedding_add: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_dyt_norm(const float* x, const float* w, const float* b, const float* alpha, void* out, const int* rows,
                             int n_rows, int hidden, int out_dtype, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && hidden > 0, "dyt_norm: empty input (%d rows, width %d)", n_rows, hidden);
  cudaStream_t s = (cudaStream_t)stream;
  TLLM_REQUIRE(out_dtype == TLLM_F32 || out_dtype == TLLM_BF16, "dyt_norm: unknown dtype code %d", out_dtype);
  if (hidden % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)b % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int n4 = hidden / 4;
    const int vthreads = n4 >= 256 ? 256 : (n4 >= 128 ? 128 : 64);
    const int per = n_rows >= 148 * 16 ? 4 : 1;
    const int blocks = (n_rows + per - 1) / per;
    if (out_dtype == TLLM_F32)
      TLLM_LAUNCH("dyt_norm", dyt_norm_vec_kernel<float>, blocks, vthreads, 0, s, x, w, b, alpha, (float*)out, rows, n_rows, hidden, per);
    else
      TLLM_LAUNCH("dyt_norm", dyt_norm_vec_kernel<__nv_bfloat16>, blocks, vthreads, 0, s, x, w, b, alpha, (__nv_bfloat16*)out, rows, n_rows, hidden, per);
    return TLLM_OK;
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == TLLM_F32)
    TLLM_LAUNCH("dyt_norm", dyt_norm_kernel<float>, n_rows, threads, 0, s, x, w, b, alpha, (float*)out, rows, n_rows, hidden);
  else if (out_dtype == TLLM_BF16)
    TLLM_LAUNCH("dyt_norm", dyt_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, s, x, w, b, alpha, (__nv_bfloat16*)out, rows, n_rows, hidden);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "dyt_norm: unknown dtype code %d", out_dtype);
  return TLLM_OK;
}

extern "C" int tllm_rope_pairs_kv_write(void* qkv, const int* positions, const float* freq, int rot_dims, int n_tokens,
                                        int nq, int nk, int nv, int kd, int vd, int row_stride, void* kcache, void* vcache,
                                        const int* slot_mapping, int page_size, long long k_page_stride,
                                        long long k_head_stride, long long v_page_stride, long long v_head_stride,
                                        int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nk > 0 && nv > 0 && vd > 0, "rope_pairs_kv_write: empty input");
  TLLM_REQUIRE(kd > 0, "rope_pairs_kv_write: key size %d", kd);
  TLLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= kd && rot_dims <= 512 && (rot_dims == 0 || freq),
               "rope_pairs_kv_write: %d rotated values of %d (even, at most the key size and 512, with a frequency table)", rot_dims, kd);
  TLLM_REQUIRE(kcache && vcache && slot_mapping && page_size > 0, "rope_pairs_kv_write: needs cache pointers, a slot mapping and a page size");
  const int work = (nq + nk) * ((kd + 1) / 2);
  const int threads = work >= 512 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("rope_pairs_kv_write", rope_pairs_kv_write_kernel<float>, n_tokens, threads, 0, s, (float*)qkv, positions, freq, rot_dims, n_tokens, nq, nk, nv, kd, vd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("rope_pairs_kv_write", rope_pairs_kv_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (__nv_bfloat16*)qkv, positions, freq, rot_dims, n_tokens, nq, nk, nv, kd, vd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "rope_pairs_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_diff_combine(const float* a, const float* lq1, const float* lk1, const float* lq2, const float* lk2,
                                 int kd, float diff, float eps, void* out, long long n_rows, int vd, int out_dtype,
                                 void* stream) {
  TLLM_REQUIRE(n_rows > 0 && vd > 0 && vd <= 256 && kd > 0, "diff_combine: %lld rows of %d values (at most 256), key size %d", n_rows, vd, kd);
  const int warps = 4;
  const long long blocks = (n_rows + warps - 1) / warps;
  TLLM_REQUIRE(blocks <= 2147483647LL, "diff_combine: %lld rows exceed the grid", n_rows);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == TLLM_F32)
    TLLM_LAUNCH("diff_combine", diff_combine_kernel<float>, (unsigned)blocks, warps * 32, 0, s, a, lq1, lk1, lq2, lk2, kd, diff, eps, (float*)out, n_rows, vd);
  else if (out_dtype == TLLM_BF16)
    TLLM_LAUNCH("diff_combine", diff_combine_kernel<__nv_bfloat16>, (unsigned)blocks, warps * 32, 0, s, a, lq1, lk1, lq2, lk2, kd, diff, eps, (__nv_bfloat16*)out, n_rows, vd);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "diff_combine: unknown dtype code %d", out_dtype);
  return TLLM_OK;
}

extern "C" int tllm_embedding(const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                              int dtype, float scale, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && hidden > 0, "embedding: empty input (%d tokens, width %d)", n_tokens, hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("embedding", embedding_kernel<float>, n_tokens, threads, 0, s, tokens, (const float*)table, out, n_tokens, hidden, scale);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("embedding", embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, tokens, (const __nv_bfloat16*)table, out, n_tokens, hidden, scale);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "embedding: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_rms_norm(const float* x, const float* w, void* out, const int* rows, int n_rows, int hidden,
                             float eps, int out_dtype, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && hidden > 0, "rms_norm: empty input (%d rows, width %d)", n_rows, hidden);
  TLLM_REQUIRE(out_dtype == TLLM_F32 || out_dtype == TLLM_BF16, "rms_norm: unknown dtype code %d", out_dtype);
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = hidden % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0;
  if (aligned && hidden <= 4 * 4 * 256) {
    // 128 or 256 threads, up to four 16-byte loads each
    const int n4 = hidden / 4;
    // Few rows (decode): more threads per row, fewer loads per thread in a row.  Only for bfloat16 output:
    // the 32-bit path promises sums whose order does not depend on what else is in the batch.
    const bool wide = out_dtype == TLLM_BF16 && n_rows <= 64;
    const int threads = wide ? (n4 <= 128 ? 128 : (n4 <= 256 ? 256 : 512)) : (n4 <= 128 * 4 ? 128 : 256);
    const int vec = (n4 + threads - 1) / threads;
#define TLLM_NORM_CASE(V)                                                                                                   \
  if (out_dtype == TLLM_F32)                                                                                               \
    TLLM_LAUNCH("rms_norm", (rms_norm_vec_kernel<float, V>), n_rows, threads, 0, s, x, w, (float*)out, rows, n_rows, hidden, eps); \
  else                                                                                                                     \
    TLLM_LAUNCH("rms_norm", (rms_norm_vec_kernel<__nv_bfloat16, V>), n_rows, threads, 0, s, x, w, (__nv_bfloat16*)out, rows, n_rows, hidden, eps); \
  return TLLM_OK;
    if (vec <= 1) { TLLM_NORM_CASE(1) }
    if (vec == 2) { TLLM_NORM_CASE(2) }
    if (vec == 3) { TLLM_NORM_CASE(3) }
    { TLLM_NORM_CASE(4) }
#undef TLLM_NORM_CASE
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == TLLM_F32)
    TLLM_LAUNCH("rms_norm", rms_norm_kernel<float>, n_rows, threads, 0, s, x, w, (float*)out, rows, n_rows, hidden, eps);
  else
    TLLM_LAUNCH("rms_norm", rms_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, s, x, w, (__nv_bfloat16*)out, rows, n_rows, hidden, eps);
  return TLLM_OK;
}

extern "C" int tllm_rms_norm_add(float* x, const float* w, float* resid, int n_rows, int hidden, float eps, float scale,
                                 int clear, void* copy_bf16, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && hidden > 0, "rms_norm_add: empty input");
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  TLLM_LAUNCH("rms_norm_add", rms_norm_add_kernel, n_rows, threads, 0, (cudaStream_t)stream, x, w, resid, n_rows, hidden, eps, scale, clear,
              (__nv_bfloat16*)copy_bf16);
  return TLLM_OK;
}

// in_dtype: dtype of `gu`; out_dtype: dtype of `out`.  zero_src != 0 (float32 `gu` only): `gu` is a
// split-K accumulation buffer and is handed back cleared.
extern "C" int tllm_silu_mul(void* gu, void* out, int m, int inter, int blk, int in_dtype, int out_dtype, int zero_src,
                             int act, void* stream) {
  TLLM_REQUIRE(m > 0 && inter > 0 && blk > 0 && inter % blk == 0,
               "silu_mul: %d rows, width %d, block %d (the block must divide the width)", m, inter, blk);
  const size_t total = (size_t)m * inter;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == TLLM_F32 && blk % 4 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0 && (out_dtype == TLLM_F32 || out_dtype == TLLM_BF16)) {
    const size_t quads = total / 4;
    const int vblocks = (int)((quads + threads - 1) / threads < 148 * 16 ? (quads + threads - 1) / threads : 148 * 16);
    if (out_dtype == TLLM_F32 && zero_src) TLLM_LAUNCH("silu_mul", (silu_mul_f32x4_kernel<float, true>), vblocks, threads, 0, s, (float*)gu, (float*)out, m, inter, blk, act);
    else if (out_dtype == TLLM_F32) TLLM_LAUNCH("silu_mul", (silu_mul_f32x4_kernel<float, false>), vblocks, threads, 0, s, (float*)gu, (float*)out, m, inter, blk, act);
    else if (zero_src) TLLM_LAUNCH("silu_mul", (silu_mul_f32x4_kernel<__nv_bfloat16, true>), vblocks, threads, 0, s, (float*)gu, (__nv_bfloat16*)out, m, inter, blk, act);
    else TLLM_LAUNCH("silu_mul", (silu_mul_f32x4_kernel<__nv_bfloat16, false>), vblocks, threads, 0, s, (float*)gu, (__nv_bfloat16*)out, m, inter, blk, act);
    return TLLM_OK;
  }
  if (in_dtype == TLLM_F32 && out_dtype == TLLM_F32 && !zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, float, false>), blocks, threads, 0, s, (float*)gu, (float*)out, m, inter, blk, act);
  else if (in_dtype == TLLM_BF16 && out_dtype == TLLM_BF16 && !zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<__nv_bfloat16, __nv_bfloat16, false>), blocks, threads, 0, s, (__nv_bfloat16*)gu, (__nv_bfloat16*)out, m, inter, blk, act);
  else if (in_dtype == TLLM_F32 && out_dtype == TLLM_BF16 && zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, __nv_bfloat16, true>), blocks, threads, 0, s, (float*)gu, (__nv_bfloat16*)out, m, inter, blk, act);
  else if (in_dtype == TLLM_F32 && out_dtype == TLLM_BF16 && !zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, __nv_bfloat16, false>), blocks, threads, 0, s, (float*)gu, (__nv_bfloat16*)out, m, inter, blk, act);
  else if (in_dtype == TLLM_F32 && out_dtype == TLLM_F32 && zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, float, true>), blocks, threads, 0, s, (float*)gu, (float*)out, m, inter, blk, act);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "silu_mul: dtype codes %d -> %d with zero_src %d are not built", in_dtype, out_dtype, zero_src);
  return TLLM_OK;
}

// `src` (optional): float32 rows of src_stride values to read instead of `qkv`; they are handed back
// zeroed (a split-K accumulation buffer); the rotated queries are written to `qkv` all the same.
extern "C" int tllm_rope_kv_write(void* qkv, float* src, int src_stride, const int* positions, const float* cos_t,
                                  const float* sin_t, int rot_dim, int n_tokens, int nq, int nkv, int hd, int row_stride,
                                  void* kcache, void* vcache, const int* slot_mapping, int page_size,
                                  long long page_stride, long long head_stride, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0, "rope_kv_write: empty input");
  TLLM_REQUIRE(hd > 0 && hd % 2 == 0, "rope_kv_write: head size %d must be even", hd);
  TLLM_REQUIRE(rot_dim == 0 || (cos_t && sin_t), "rope_kv_write: rotary size %d without tables", rot_dim);
  TLLM_REQUIRE(rot_dim == 0 || rot_dim == hd, "rope_kv_write: partial rotary (%d of %d dims) is not built", rot_dim, hd);
  TLLM_REQUIRE(!slot_mapping || (kcache && vcache && page_size > 0), "rope_kv_write: a slot mapping needs cache pointers and a page size");
  const int work = (nq + nkv) * hd / 2;
  const int threads = work >= 512 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  const float* c = rot_dim ? cos_t : nullptr;
  const float* sn = rot_dim ? sin_t : nullptr;
  const int esz = dtype == TLLM_F32 ? 4 : 2;
  const bool vec = hd % 16 == 0 && ((uintptr_t)qkv % 16) == 0 && ((long long)row_stride * esz) % 16 == 0 &&
                   (!src || (((uintptr_t)src % 16) == 0 && src_stride % 4 == 0)) &&
                   (!slot_mapping || (((uintptr_t)kcache % 16) == 0 && ((uintptr_t)vcache % 16) == 0 &&
                                      (page_stride * esz) % 16 == 0 && (head_stride * esz) % 16 == 0)) &&
                   (!c || (((uintptr_t)c % 16) == 0 && ((uintptr_t)sn % 16) == 0));
  if (vec) {
    const int items = (nq + nkv) * (hd / 16);
    const int vthreads = items >= 256 ? 256 : 128;
    // few tokens: up to four CTAs per token, so that no thread walks its items one after the other
    const int parts = n_tokens <= 256 ? std::min(4, (items + vthreads - 1) / vthreads) : 1;
    const dim3 vgrid((unsigned)n_tokens, (unsigned)parts);
    if (dtype == TLLM_F32)
      TLLM_LAUNCH("rope_kv_write", rope_kv_write_vec_kernel<float>, vgrid, vthreads, 0, s, (float*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, page_stride, head_stride);
    else if (dtype == TLLM_BF16)
      TLLM_LAUNCH("rope_kv_write", rope_kv_write_vec_kernel<__nv_bfloat16>, vgrid, vthreads, 0, s, (__nv_bfloat16*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, page_stride, head_stride);
    else
      TLLM_FAIL(TLLM_ERR_ARG, "rope_kv_write: unknown dtype code %d", dtype);
    return TLLM_OK;
  }
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("rope_kv_write", rope_kv_write_kernel<float>, n_tokens, threads, 0, s, (float*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, page_stride, head_stride);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("rope_kv_write", rope_kv_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (__nv_bfloat16*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, page_stride, head_stride);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "rope_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}

// ---------------------------------------------------------------- hashed bigram rows added into the stream
// out[t, :] += table[row_t, :] with row_t = (prev_t * mul_prev + tokens[t] * mul_cur) mod buckets, prev_t the token
// before t in its sequence; a sequence's first token takes row `buckets`.  The token before a step's first one is
// the request's state (`last` [slots] int32), which the CTA of the request's first token of the step reads and then
// replaces by the request's last token of the step: one launch, one reader and one writer per slot.
namespace tllm {
template <typename T>
__global__ void bigram_add_kernel(const int* __restrict__ tokens, const int* __restrict__ token_request,
                                  const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                  const int* __restrict__ slots, int* __restrict__ last, const T* __restrict__ table,
                                  float* __restrict__ out, int n_tokens, int hidden, long long buckets,
                                  long long mul_prev, long long mul_cur) {
  __shared__ long long s_row;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  if (threadIdx.x == 0) {
    const int req = token_request[t];
    const int first = cu_q[req];
    long long row = buckets;
    if (t > first) {
      row = ((long long)tokens[t - 1] * mul_prev + (long long)tokens[t] * mul_cur) % buckets;
    } else {
      int* slot = last + slots[req];
      if (q_start[req] > 0) row = ((long long)*slot * mul_prev + (long long)tokens[t] * mul_cur) % buckets;
      *slot = tokens[cu_q[req + 1] - 1];
    }
    s_row = row;
  }
  __syncthreads();
  const T* src = table + (size_t)s_row * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] += to_f32(src[i]);
}

// ---------------------------------------------------------------- element by element: a copy in another type, or relu(x)^2
template <typename TI, typename TO>
__global__ void unary_kernel(const TI* __restrict__ x, TO* __restrict__ out, long long n, int act) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = to_f32(x[i]);
    if (act == 1) { v = fmaxf(v, 0.f); v = __fmul_rn(v, v); }
    out[i] = from_f32<TO>(v);
  }
}

// resid += scale * x, element by element in 32-bit; clear != 0 hands x back zeroed
__global__ void scaled_add_kernel(float* __restrict__ x, float* __restrict__ resid, long long n, float scale, int clear) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    resid[i] = fmaf(scale, x[i], resid[i]);
    if (clear) x[i] = 0.f;
  }
}
}  // namespace tllm

extern "C" int tllm_bigram_add(const int* tokens, const int* token_request, const int* cu_q, const int* q_start,
                               const int* slots, int* last, const void* table, float* out, int n_tokens, int hidden,
                               long long buckets, long long mul_prev, long long mul_cur, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && hidden > 0 && buckets > 0, "bigram_add: %d tokens, width %d, %lld buckets", n_tokens, hidden, buckets);
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("bigram_add", bigram_add_kernel<float>, n_tokens, threads, 0, s, tokens, token_request, cu_q, q_start, slots, last, (const float*)table, out, n_tokens, hidden, buckets, mul_prev, mul_cur);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("bigram_add", bigram_add_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, tokens, token_request, cu_q, q_start, slots, last, (const __nv_bfloat16*)table, out, n_tokens, hidden, buckets, mul_prev, mul_cur);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "bigram_add: unknown dtype code %d", dtype);
  return TLLM_OK;
}

// act: 0 = the value as it is (a copy in the output's type), 1 = relu(x)^2
extern "C" int tllm_unary(const void* x, void* out, long long n, int in_dtype, int out_dtype, int act, void* stream) {
  TLLM_REQUIRE(n > 0 && (act == 0 || act == 1), "unary: %lld values, activation code %d", n, act);
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == TLLM_F32 && out_dtype == TLLM_F32)
    TLLM_LAUNCH("unary", (unary_kernel<float, float>), blocks, threads, 0, s, (const float*)x, (float*)out, n, act);
  else if (in_dtype == TLLM_F32 && out_dtype == TLLM_BF16)
    TLLM_LAUNCH("unary", (unary_kernel<float, __nv_bfloat16>), blocks, threads, 0, s, (const float*)x, (__nv_bfloat16*)out, n, act);
  else if (in_dtype == TLLM_BF16 && out_dtype == TLLM_BF16)
    TLLM_LAUNCH("unary", (unary_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, threads, 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, act);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "unary: dtype codes %d -> %d are not built", in_dtype, out_dtype);
  return TLLM_OK;
}

extern "C" int tllm_scaled_add(float* x, float* resid, long long n, float scale, int clear, void* stream) {
  TLLM_REQUIRE(n > 0, "scaled_add: empty input");
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  TLLM_LAUNCH("scaled_add", scaled_add_kernel, blocks, threads, 0, (cudaStream_t)stream, x, resid, n, scale, clear);
  return TLLM_OK;
}
