// Linear attention with a matrix state per head, carried from step to step in 32-bit:
//   S_t = diag(a_t) S_(t-1) + (ks k_t) v_t^T,   o_t = S_t^T (qs q_t)        S: [key size, value size]
// The decay a_t is either one constant per head (retention) or one number per key channel and token,
//   a = sigmoid(z + b)^(1/tau) = exp(-softplus(-(z + b)) / tau)             (gated linear attention)
// with z the 32-bit rows of a projection.  Decays, the recurrence and the state are 32-bit; q, k, v are projection
// outputs of the engine's dtype.  The state of a request lives in state[slot, head, key, value] and is read at the
// start of the request's tokens in the step and written back after the last one.
//
// scan: a CTA owns 64 value columns of one (request, head); a thread owns 16 state rows of two columns in registers.
// Eight tokens at a time are staged in shared memory (scaled queries and keys, decays); every thread walks them,
// leaves its partial dot products, and the partials of a column are added over the row slices in a fixed order.
// The operations on a state element are those of the sequence, whatever the cut into steps: the same bits.
//
// SEGMENTED (long portions): the tokens of a request are cut into segments; a first kernel walks every segment from
// a zero state and keeps its end state and the product of its decays per row (S_end = diag(A) S_in + B); a small
// kernel walks each request's summaries in order and leaves every segment's S_in in their place; a third walks the
// segments again from there, now writing outputs.  The recurrence is linear in S, so the two ways differ by rounding only.
//
// head_norm_gate: y = o / sqrt(mean(o^2) + eps) * w * silu(g) (or sigmoid(g)) per (token, head), 32-bit in, engine dtype out.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int LA_ROWS = 16;   // state rows per thread
constexpr int LA_CPT = 2;     // value columns per thread (lane and lane + 32)
constexpr int LA_COLS = 32 * LA_CPT;   // value columns per CTA
constexpr int LA_TOK = 8;     // tokens staged at once

__device__ __forceinline__ float gate_decay(float x, float inv_tau) {
  // sigmoid(x)^(1/tau) without forming the sigmoid: exp(-softplus(-x) / tau)
  const float sp = fmaxf(-x, 0.f) + log1pf(expf(-fabsf(x)));
  return expf(-sp * inv_tau);
}

struct ScanArgs {
  const void *q, *k, *v;
  int ldq, ldk, ldv;
  const float* head_decay;   // [heads] or null
  const float* gate;         // [T, heads * kd] rows of ldg values, or null
  int ldg;
  const float* gate_bias;    // [heads * kd]
  float inv_tau, q_scale, k_scale;
  float* state;              // [slots, heads, kd, vd]
  const int* slots;
  const int* cu_q;
  float* out;                // [T, heads * vd]
  int heads, kd, vd;
  // segments: 0 = serial
  int seg, max_segs;
  float* summary;            // [requests, max_segs, heads, (kd * vd) + kd]
};

// mode 0: serial over the request's tokens, from and to `state`.
// mode 1: a segment from a zero state; writes the end state and the decay products to `summary` (no outputs).
// mode 2: a segment from the state that the prefix kernel left in `summary`; writes outputs, and the last
//         segment of a request the state.
// GATED: a decay per key channel and token (staged with the queries and keys); else one per head.
template <typename T, int MODE, bool GATED>
__global__ void __launch_bounds__(512) linear_attention_scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  const int lane = threadIdx.x, sl = threadIdx.y, nsl = blockDim.y;
  const int kdp = nsl * LA_ROWS;
  float* sq = sm;                       // [LA_TOK][kdp]
  float* sk = sq + LA_TOK * kdp;        // [LA_TOK][kdp]
  float* sa = sk + LA_TOK * kdp;        // [LA_TOK][kdp]
  float* part = sa + LA_TOK * kdp;      // [LA_TOK][nsl][LA_COLS]
  const int h = blockIdx.y;
  const int r = MODE == 0 ? blockIdx.z : blockIdx.z / a.max_segs;
  const int sg = MODE == 0 ? 0 : blockIdx.z % a.max_segs;
  int col[LA_CPT];
  bool col_ok[LA_CPT];
#pragma unroll
  for (int c = 0; c < LA_CPT; ++c) {
    col[c] = blockIdx.x * LA_COLS + c * 32 + lane;
    col_ok[c] = col[c] < a.vd;
  }
  const int tid = sl * 32 + lane, nthreads = nsl * 32;
  const float hd = GATED ? 1.f : a.head_decay[h];
  pdl_wait();
  int t0 = a.cu_q[r], t1 = a.cu_q[r + 1];
  if (MODE != 0) {
    t0 += sg * a.seg;
    t1 = min(t1, t0 + a.seg);
    if (t0 >= t1) return;
  }
  const bool last = t1 == a.cu_q[r + 1];
  if (MODE == 1 && last) return;   // the last segment's summary is never read
  const T* q = (const T*)a.q;
  const T* k = (const T*)a.k;
  const T* v = (const T*)a.v;
  float* st = a.state + (((size_t)a.slots[r] * a.heads + h) * a.kd) * a.vd;
  const size_t per = (size_t)a.kd * a.vd + a.kd;
  float* su = MODE == 0 ? nullptr : a.summary + (((size_t)r * a.max_segs + sg) * a.heads + h) * per;
  float s[LA_CPT][LA_ROWS];
  float dprod[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int row = sl * LA_ROWS + i;
    dprod[i] = 1.f;
#pragma unroll
    for (int c = 0; c < LA_CPT; ++c) {
      const bool ok = col_ok[c] && row < a.kd;
      if (MODE == 0) s[c][i] = ok ? st[(size_t)row * a.vd + col[c]] : 0.f;
      else if (MODE == 1) s[c][i] = 0.f;
      else s[c][i] = ok ? su[(size_t)row * a.vd + col[c]] : 0.f;
    }
  }
  // The next tile's values are fetched into registers while the current tile is walked: NST staged elements of
  // each of q, k (and the gate) and LA_TOK values of each column per thread.
  constexpr int NST = LA_TOK * LA_ROWS / 32;
  float rq[NST], rk[NST], rz[NST], vn[LA_CPT][LA_TOK];
  auto fetch = [&](int tb) {
    const int nt = min(LA_TOK, t1 - tb);
#pragma unroll
    for (int x = 0; x < NST; ++x) {
      const int idx = tid + x * nthreads;
      const int tt = idx / kdp, row = idx % kdp;
      rq[x] = rk[x] = rz[x] = 0.f;
      if (tt < nt && row < a.kd) {
        const size_t t = (size_t)(tb + tt);
        rq[x] = to_f32(q[t * a.ldq + h * a.kd + row]);
        rk[x] = to_f32(k[t * a.ldk + h * a.kd + row]);
        if (GATED) rz[x] = a.gate[t * a.ldg + h * a.kd + row] + a.gate_bias[h * a.kd + row];
      }
    }
#pragma unroll
    for (int tt = 0; tt < LA_TOK; ++tt)
#pragma unroll
      for (int c = 0; c < LA_CPT; ++c)
        vn[c][tt] = (tt < nt && col_ok[c]) ? to_f32(v[(size_t)(tb + tt) * a.ldv + h * a.vd + col[c]]) : 0.f;
  };
  fetch(t0);
  for (int tb = t0; tb < t1; tb += LA_TOK) {
    const int nt = min(LA_TOK, t1 - tb);
#pragma unroll
    for (int x = 0; x < NST; ++x) {
      const int idx = tid + x * nthreads;
      const int tt = idx / kdp, row = idx % kdp;
      const bool in = tt < nt && row < a.kd;
      sq[idx] = rq[x] * a.q_scale;
      sk[idx] = rk[x] * a.k_scale;
      if (GATED) sa[idx] = in ? gate_decay(rz[x], a.inv_tau) : 1.f;
    }
    float vv[LA_CPT][LA_TOK];
#pragma unroll
    for (int tt = 0; tt < LA_TOK; ++tt)
#pragma unroll
      for (int c = 0; c < LA_CPT; ++c) vv[c][tt] = vn[c][tt];
    __syncthreads();
    if (tb + LA_TOK < t1) fetch(tb + LA_TOK);
#pragma unroll
    for (int tt = 0; tt < LA_TOK; ++tt) {
      if (tt < nt) {
        const float4* pq = reinterpret_cast<const float4*>(sq + tt * kdp + sl * LA_ROWS);
        const float4* pk = reinterpret_cast<const float4*>(sk + tt * kdp + sl * LA_ROWS);
        const float4* pa = reinterpret_cast<const float4*>(sa + tt * kdp + sl * LA_ROWS);
        float acc[LA_CPT];
#pragma unroll
        for (int c = 0; c < LA_CPT; ++c) acc[c] = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < LA_ROWS / 4; ++i4) {
          const float4 q4 = pq[i4], k4 = pk[i4];
          const float4 a4 = GATED ? pa[i4] : make_float4(hd, hd, hd, hd);
          const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = i4 * 4 + x;
            if (MODE == 1) dprod[i] *= aa[x];
#pragma unroll
            for (int c = 0; c < LA_CPT; ++c) {
              s[c][i] = fmaf(aa[x], s[c][i], ka[x] * vv[c][tt]);
              acc[c] = fmaf(s[c][i], qa[x], acc[c]);
            }
          }
        }
        if (MODE != 1) {
#pragma unroll
          for (int c = 0; c < LA_CPT; ++c) part[(tt * nsl + sl) * LA_COLS + c * 32 + lane] = acc[c];
        }
      }
    }
    __syncthreads();
    if (MODE != 1) {
      for (int idx = tid; idx < nt * LA_COLS; idx += nthreads) {
        const int tt = idx / LA_COLS, c = idx % LA_COLS;
        const int oc = blockIdx.x * LA_COLS + c;
        if (oc < a.vd) {
          float o = 0.f;
          for (int x = 0; x < nsl; ++x) o += part[(tt * nsl + x) * LA_COLS + c];
          a.out[(size_t)(tb + tt) * a.heads * a.vd + h * a.vd + oc] = o;
        }
      }
    }
  }
  if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < LA_ROWS; ++i) {
      const int row = sl * LA_ROWS + i;
      if (row < a.kd) {
#pragma unroll
        for (int c = 0; c < LA_CPT; ++c)
          if (col_ok[c]) su[(size_t)row * a.vd + col[c]] = s[c][i];
        if (col[0] == 0) su[(size_t)a.kd * a.vd + row] = dprod[i];
      }
    }
  } else if (MODE == 0 || last) {
#pragma unroll
    for (int i = 0; i < LA_ROWS; ++i) {
      const int row = sl * LA_ROWS + i;
#pragma unroll
      for (int c = 0; c < LA_CPT; ++c)
        if (col_ok[c] && row < a.kd) st[(size_t)row * a.vd + col[c]] = s[c][i];
    }
  }
}

// Between the two passes over the segments: every state element walks its request's summaries in order and leaves,
// in place of each segment's end state B_g, the state the segment starts from: x_0 = the carried state,
// x_(g+1) = A_g x_g + B_g.  (The last segment's own summary was not written and is not read.)
__global__ void linear_attention_prefix_kernel(ScanArgs a) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, r = blockIdx.z;
  const int len = a.cu_q[r + 1] - a.cu_q[r];
  const int nseg = (len + a.seg - 1) / a.seg;
  const size_t per = (size_t)a.kd * a.vd + a.kd;
  const float* st = a.state + (((size_t)a.slots[r] * a.heads + h) * a.kd) * a.vd;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < a.kd * a.vd; e += gridDim.x * blockDim.x) {
    const int row = e / a.vd;
    float x = st[e];
    // eight segments' summaries are fetched before the first of them is overwritten
    for (int g0 = 0; g0 < nseg; g0 += 8) {
      float b[8], d[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int g = g0 + u;
        const bool more = g + 1 < nseg;
        const float* su = a.summary + (((size_t)r * a.max_segs + (more ? g : 0)) * a.heads + h) * per;
        b[u] = more ? su[e] : 0.f;
        d[u] = more ? su[(size_t)a.kd * a.vd + row] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int g = g0 + u;
        if (g < nseg) {
          a.summary[(((size_t)r * a.max_segs + g) * a.heads + h) * per + e] = x;
          x = fmaf(d[u], x, b[u]);
        }
      }
    }
  }
}

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ g,
                                      int ldg, int heads, int vd, float eps, T* __restrict__ out, long long n_rows, int act) {
  pdl_trigger();
  pdl_wait();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int h = (int)(row % heads);
  const float* x = o + row * vd;
  float ss = 0.f;
  for (int j = lane; j < vd; j += 32) ss = fmaf(x[j], x[j], ss);
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)vd + eps);
  const T* gr = g + t * ldg + (size_t)h * vd;
  T* y = out + row * vd;
  for (int j = lane; j < vd; j += 32) {
    const float gv = to_f32(gr[j]);
    const float sg = (act == 1 ? 1.f : gv) / (1.f + expf(-gv));   // act 1: sigmoid, else silu
    float val = x[j] * r;
    if (w) val *= w[j];
    y[j] = from_f32<T>(val * sg);
  }
}

}  // namespace tllm

using namespace tllm;

// q, k: [T, heads * kd] rows of ldq / ldk values; v: [T, heads * vd] rows of ldv values (dtype: 0 float32, 1 bfloat16).
// Exactly one of head_decay (float32 [heads]) and gate (float32 [T, heads * kd] rows of ldg values, with gate_bias
// [heads * kd] and inv_tau) is given.  out: float32 [T, heads * vd].  seg > 0: segments of that many tokens with
// `summary` (float32, n_requests * max_segs * heads * (kd * vd + kd) values); seg = 0: serial.
extern "C" int tllm_linear_attention_scan(const void* q, const void* k, const void* v, int ldq, int ldk, int ldv,
                                          const float* head_decay, const float* gate, int ldg, const float* gate_bias,
                                          float inv_tau, float q_scale, float k_scale, float* state, const int* slots,
                                          const int* cu_q, float* out, int heads, int kd, int vd, int n_requests,
                                          int max_q_len, int seg, float* summary, int dtype, void* stream) {
  TLLM_REQUIRE(heads > 0 && kd > 0 && vd > 0 && n_requests > 0 && max_q_len > 0, "linear_attention_scan: empty input");
  TLLM_REQUIRE(kd <= 256, "linear_attention_scan: key size %d (at most 256)", kd);
  TLLM_REQUIRE((head_decay != nullptr) != (gate != nullptr), "linear_attention_scan: one of a decay per head and a gate");
  TLLM_REQUIRE(!gate || gate_bias, "linear_attention_scan: a gate needs its bias");
  TLLM_REQUIRE(dtype == TLLM_F32 || dtype == TLLM_BF16, "linear_attention_scan: unknown dtype code %d", dtype);
  TLLM_REQUIRE(heads <= 65535, "linear_attention_scan: %d heads exceed the grid", heads);
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.ldq = ldq; a.ldk = ldk; a.ldv = ldv;
  a.head_decay = head_decay; a.gate = gate; a.ldg = ldg; a.gate_bias = gate_bias;
  a.inv_tau = inv_tau; a.q_scale = q_scale; a.k_scale = k_scale;
  a.state = state; a.slots = slots; a.cu_q = cu_q; a.out = out; a.heads = heads; a.kd = kd; a.vd = vd;
  a.seg = 0; a.max_segs = 1; a.summary = nullptr;
  const int nsl = (kd + LA_ROWS - 1) / LA_ROWS;
  const dim3 block(32, nsl);
  const size_t smem = (size_t)(3 * LA_TOK * nsl * LA_ROWS + LA_TOK * nsl * LA_COLS) * sizeof(float);
  const unsigned bx = (unsigned)((vd + LA_COLS - 1) / LA_COLS);
  cudaStream_t s = (cudaStream_t)stream;
  const bool gated = gate != nullptr;
#define TLLM_SCAN(name, T, MODE)                                                                          \
  do {                                                                                                    \
    if (gated) TLLM_LAUNCH(name, (linear_attention_scan_kernel<T, MODE, true>), grid, block, smem, s, a);  \
    else TLLM_LAUNCH(name, (linear_attention_scan_kernel<T, MODE, false>), grid, block, smem, s, a);       \
  } while (0)
  if (seg <= 0 || max_q_len <= seg) {
    TLLM_REQUIRE(n_requests <= 65535, "linear_attention_scan: %d requests exceed the grid", n_requests);
    const dim3 grid(bx, (unsigned)heads, (unsigned)n_requests);
    if (dtype == TLLM_F32) TLLM_SCAN("linear_attention_scan", float, 0);
    else TLLM_SCAN("linear_attention_scan", __nv_bfloat16, 0);
    return TLLM_OK;
  }
  TLLM_REQUIRE(summary != nullptr, "linear_attention_scan: segments need a summary buffer");
  a.seg = seg;
  a.max_segs = (max_q_len + seg - 1) / seg;
  TLLM_REQUIRE((long long)a.max_segs * n_requests <= 65535, "linear_attention_scan: %d segments of %d requests exceed the grid", a.max_segs, n_requests);
  a.summary = summary;
  const dim3 grid(bx, (unsigned)heads, (unsigned)(n_requests * a.max_segs));
  const dim3 pgrid((unsigned)((kd * vd + 255) / 256), (unsigned)heads, (unsigned)n_requests);
  if (dtype == TLLM_F32) TLLM_SCAN("linear_attention_summary", float, 1);
  else TLLM_SCAN("linear_attention_summary", __nv_bfloat16, 1);
  TLLM_LAUNCH("linear_attention_prefix", linear_attention_prefix_kernel, pgrid, 256, 0, s, a);
  if (dtype == TLLM_F32) TLLM_SCAN("linear_attention_segments", float, 2);
  else TLLM_SCAN("linear_attention_segments", __nv_bfloat16, 2);
#undef TLLM_SCAN
  return TLLM_OK;
}

// o: float32 [n_rows = T * heads, vd]; w: float32 [vd] or null; g: [T, heads * vd] rows of ldg values; out: [T, heads * vd].
extern "C" int tllm_head_norm_gate(const float* o, const float* w, const void* g, int ldg, int heads, int vd, float eps,
                                   void* out, long long n_rows, int dtype, int act, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && heads > 0 && vd > 0, "head_norm_gate: empty input");
  const int warps = 4;
  const long long blocks = (n_rows + warps - 1) / warps;
  TLLM_REQUIRE(blocks <= 2147483647LL, "head_norm_gate: %lld rows exceed the grid", n_rows);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("head_norm_gate", head_norm_gate_kernel<float>, (unsigned)blocks, warps * 32, 0, s, o, w, (const float*)g, ldg, heads, vd, eps, (float*)out, n_rows, act);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("head_norm_gate", head_norm_gate_kernel<__nv_bfloat16>, (unsigned)blocks, warps * 32, 0, s, o, w, (const __nv_bfloat16*)g, ldg, heads, vd, eps, (__nv_bfloat16*)out, n_rows, act);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "head_norm_gate: unknown dtype code %d", dtype);
  return TLLM_OK;
}
