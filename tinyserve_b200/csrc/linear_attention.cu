// Linear attention with a decaying matrix state, for one key size per build (-DTS_KEY_DIM=...):
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: key size x value size, per request and head)
//   o_t = S_t^T q_t
//
// a_t is either one constant per head (retention: `decay`) or one number per key channel and
// token, a_t = sigmoid(z_t)^(1 / tau) (gated linear attention: `z` holds the 32-bit logits).
// q and k may get rotary positions on their first rotary_dim elements and a constant factor
// each.  The head's output is divided by its root mean square over the value size (times an
// optional weight), multiplied by silu(gate) and stored as T for the output projection.
//
// The state is 32-bit, lives in the request's state slot between steps, and starts at zero for
// a request whose first token is in this step.  Everything after the projections is 32-bit
// arithmetic: angles, decays, the state, the output norm.  T is the storage type of the
// projections, the gate and the result (float or bfloat16).
//
// One block per (request, head) walks the request's tokens of this step in order, a single
// decoded token and a prompt portion of any length alike.  (A head of more than 128 value
// columns is spread over several blocks of 128 columns; the output norm, which needs the whole
// head, then runs as a kernel of its own on the 32-bit outputs.)  Thread (column c, row group g) keeps
// rows [g R, (g + 1) R) of column c of the state in registers (R = key size / 4); the four
// groups of a column are neighbouring lanes and add their shares of o_t by shuffles.  Tokens
// are staged through shared memory sixteen at a time (rotary, factors and decays applied while
// staging), and the output norm and gate run once per sixteen tokens on the staged outputs.
//
// Long portions are cut into segments of `seg_len` tokens that run side by side (a request of
// 2,048 tokens and 8 heads alone would keep 8 of 148 SMs busy): the recurrence is linear in S, so
//   (1) every segment but a request's last runs from a zero state and leaves its local end state
//       L_p and the product D_p of its decays (SCAN_LOCAL),
//   (2) one pass over the segments turns them into start states, S_(p+1) = D_p S_p + L_p, from
//       the request's stored state (combine kernel),
//   (3) every segment runs again from its start state and makes its outputs; the last one stores
//       the request's new state (SCAN_FROM_SEGMENT).
// Nothing is divided by a decay anywhere, so no product of decays can overflow or vanish into a
// division.  Short portions and decoded tokens run as one segment in one launch (SCAN_WHOLE).
#include "common.cuh"

#ifndef TS_KEY_DIM
#error "compile with -DTS_KEY_DIM=<key size, a multiple of 4>"
#endif

TS_DEFINE_LAST_ERROR()

namespace {

constexpr int DIM = TS_KEY_DIM;
constexpr int GROUPS = 4;                 // row groups of a column
constexpr int R = DIM / GROUPS;           // state rows of a thread
constexpr int RP = R + 4;                 // padded length of a group's run in shared memory
constexpr int CHUNK = 16;                 // tokens staged at a time
static_assert(DIM % GROUPS == 0 && DIM >= 4 && DIM <= 512, "key size must be a multiple of 4 up to 512");

struct ScanParams {
  const void* q; const void* k; const void* v; const void* gate;
  long long ldq, ldk, ldv, ldg;           // row strides in elements
  const float* z; long long ldz;          // per-channel decay logits [T, H * DIM], or null
  const float* decay;                     // [H], used when z is null
  float inv_tau;
  const int* positions; const float* cos; const float* sin; int rotary_dim;
  float q_scale, k_scale;
  float* state;                           // [slots, H, DIM, vdim]
  const int* state_slots; const int* fresh; const int* cu_q;
  const void* norm_weight; int norm_weight_is_f32; float eps;
  void* out; long long ldo;               // [T, H * vdim]
  int H, vdim;
  int seg_len;                            // tokens per segment; 0: a request's tokens are one segment
  float* seg_state;                       // [B, H, segments, DIM, vdim]: local end states, then start states
  float* seg_decay;                       // [B, H, segments, DIM]: product of a segment's decays (per channel)
  int max_segments;
  int cols, col_tiles;                    // value columns per block; blocks per head
  float* raw_out;                         // [T, H * vdim] 32-bit o_t before norm and gate (col_tiles > 1), else null
};

enum { SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_FROM_SEGMENT = 2 };

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

constexpr int MAX_THREADS = 512;

template <typename T, bool PER_CHANNEL, int MODE>
__global__ void __launch_bounds__(MAX_THREADS, 1) linear_attention_scan_kernel(ScanParams p) {
  extern __shared__ float smem[];
  const int vdim = p.vdim, cols = p.cols;
  float* sq = smem;                                   // [CHUNK][GROUPS][RP]
  float* sk = sq + CHUNK * GROUPS * RP;
  float* sa = sk + CHUNK * GROUPS * RP;               // PER_CHANNEL only
  float* sv = sa + (PER_CHANNEL ? CHUNK * GROUPS * RP : 0);   // [CHUNK][cols]
  float* so = sv + CHUNK * cols;                      // [CHUNK][cols]
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x / p.col_tiles, col0 = (blockIdx.x % p.col_tiles) * cols, h = blockIdx.y, seg = blockIdx.z;
  int t0 = p.cu_q[b], t1 = p.cu_q[b + 1];
  const int request_end = t1;
  if (MODE != SCAN_WHOLE) {
    t0 += seg * p.seg_len;
    t1 = min(t1, t0 + p.seg_len);
  }
  if (t1 <= t0) return;
  const bool last = t1 == request_end;
  if (MODE == SCAN_LOCAL && last) return;          // the last segment's end state is the output pass's
  const int tid = threadIdx.x, lc = tid / GROUPS, c = col0 + lc, g = tid % GROUPS;
  const bool owner = lc < cols && c < vdim;
  const int slot = p.state_slots[b];
  float* S = p.state + (((size_t)slot * p.H + h) * DIM + (size_t)g * R) * vdim + c;
  const size_t seg_index = ((size_t)b * p.H + h) * p.max_segments + seg;
  float* seg_S = MODE == SCAN_WHOLE ? nullptr : p.seg_state + (seg_index * DIM + (size_t)g * R) * vdim + c;
  float s[R];
  float dprod[PER_CHANNEL && MODE == SCAN_LOCAL ? R : 1];
  if (PER_CHANNEL && MODE == SCAN_LOCAL) {
#pragma unroll
    for (int r = 0; r < R; ++r) dprod[r] = 1.f;
  }
  if (MODE == SCAN_WHOLE && owner && !p.fresh[b]) {
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = S[(size_t)r * vdim];
  } else if (MODE == SCAN_FROM_SEGMENT && owner) {
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = seg_S[(size_t)r * vdim];
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = 0.f;
  }
  const float head_decay = PER_CHANNEL ? 1.f : p.decay[h];
  const T* q = static_cast<const T*>(p.q) + (size_t)h * DIM;
  const T* k = static_cast<const T*>(p.k) + (size_t)h * DIM;
  const T* v = static_cast<const T*>(p.v) + (size_t)h * vdim;
  const T* gate = static_cast<const T*>(p.gate) + (size_t)h * vdim;
  T* out = static_cast<T*>(p.out) + (size_t)h * vdim;
  const int rot = p.rotary_dim, half = rot >> 1;
  VecParam nw{p.norm_weight, p.norm_weight_is_f32};
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;

  for (int base = t0; base < t1; base += CHUNK) {
    const int n = min(CHUNK, t1 - base);
    // stage q, k (rotary and factor applied), the decays and v
    for (int idx = tid; idx < n * DIM; idx += blockDim.x) {
      const int tok = idx / DIM, i = idx % DIM;
      const size_t t = base + tok;
      float qa = to_f32<T>(q[t * p.ldq + i]), ka = to_f32<T>(k[t * p.ldk + i]);
      if (i < rot) {
        const bool first = i < half;
        const int j = first ? i : i - half, mate = first ? i + half : i - half;
        const float qb = to_f32<T>(q[t * p.ldq + mate]), kb = to_f32<T>(k[t * p.ldk + mate]);
        const size_t at = (size_t)p.positions[t] * half + j;
        const float cs = p.cos[at], sn = p.sin[at];
        qa = first ? qa * cs - qb * sn : qa * cs + qb * sn;
        ka = first ? ka * cs - kb * sn : ka * cs + kb * sn;
      }
      const int where = (tok * GROUPS + i / R) * RP + i % R;
      if (MODE != SCAN_LOCAL) sq[where] = qa * p.q_scale;
      sk[where] = ka * p.k_scale;
      if (PER_CHANNEL) sa[where] = expf(log_sigmoid(p.z[t * p.ldz + (size_t)h * DIM + i]) * p.inv_tau);
    }
    for (int idx = tid; idx < n * cols; idx += blockDim.x) {
      const int tok = idx / cols, i = idx % cols;
      sv[tok * cols + i] = col0 + i < vdim ? to_f32<T>(v[(size_t)(base + tok) * p.ldv + col0 + i]) : 0.f;
    }
    __syncthreads();
    {       // (threads beyond the columns run along with a value of zero: the shuffles need whole warps)
      for (int tok = 0; tok < n; ++tok) {
        const float* qr = sq + (tok * GROUPS + g) * RP;
        const float* kr = sk + (tok * GROUPS + g) * RP;
        const float* ar = sa + (tok * GROUPS + g) * RP;
        const float vv = owner ? sv[tok * cols + lc] : 0.f;
        if (MODE == SCAN_LOCAL) {
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float a = PER_CHANNEL ? ar[r] : head_decay;
            s[r] = fmaf(a, s[r], kr[r] * vv);
            if (PER_CHANNEL && c == 0) dprod[r] *= a;      // (column 0 of the head: one block's first four threads)
          }
          continue;
        }
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float a = PER_CHANNEL ? ar[r] : head_decay;
          s[r] = fmaf(a, s[r], kr[r] * vv);
          acc = fmaf(s[r], qr[r], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (g == 0 && owner) so[tok * cols + lc] = acc;
      }
    }
    __syncthreads();
    // output norm over the value size, gate, store: a warp per token
    if constexpr (MODE != SCAN_LOCAL)
    for (int tok = warp; tok < n; tok += warps) {
      const size_t t = base + tok;
      if (p.raw_out) {            // the head spans several blocks: its norm is another kernel's
        for (int i = lane; i < cols && col0 + i < vdim; i += 32)
          p.raw_out[t * p.H * vdim + (size_t)h * vdim + col0 + i] = so[tok * cols + i];
        continue;
      }
      float acc = 0.f;
      for (int i = lane; i < vdim; i += 32) acc += so[tok * cols + i] * so[tok * cols + i];
      const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + p.eps);
      for (int i = lane; i < vdim; i += 32) {
        float o = so[tok * cols + i] * rstd;
        if (p.norm_weight) o *= nw[i];
        if (p.gate) {
          const float gv = to_f32<T>(gate[t * p.ldg + i]);
          o *= gv / (1.f + expf(-gv));
        }
        out[t * p.ldo + i] = from_f32<T>(o);
      }
    }
    if constexpr (MODE != SCAN_LOCAL) __syncthreads();
  }
  if (MODE == SCAN_LOCAL) {
    if (owner) {
#pragma unroll
      for (int r = 0; r < R; ++r) seg_S[(size_t)r * vdim] = s[r];
    }
    if (PER_CHANNEL && c == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) p.seg_decay[seg_index * DIM + g * R + r] = dprod[r];
    }
    return;
  }
  if (owner && (MODE == SCAN_WHOLE || last)) {
#pragma unroll
    for (int r = 0; r < R; ++r) S[(size_t)r * vdim] = s[r];
  }
}

// o_t of whole heads (32-bit) -> o / rms(o) (* weight) * silu(gate), stored as T: a warp per
// (token, head), for heads that the scan spread over several blocks
template <typename T>
__global__ void linear_attention_finish_kernel(ScanParams p, int num_tokens) {
  pdl_trigger();
  pdl_wait();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t t = blockIdx.x;
  const int vdim = p.vdim;
  VecParam nw{p.norm_weight, p.norm_weight_is_f32};
  for (int h = warp; h < p.H; h += warps) {
    const float* o = p.raw_out + t * p.H * vdim + (size_t)h * vdim;
    float acc = 0.f;
    for (int i = lane; i < vdim; i += 32) acc += o[i] * o[i];
    const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + p.eps);
    for (int i = lane; i < vdim; i += 32) {
      float y = o[i] * rstd;
      if (p.norm_weight) y *= nw[i];
      if (p.gate) {
        const float gv = to_f32<T>(static_cast<const T*>(p.gate)[t * p.ldg + (size_t)h * vdim + i]);
        y *= gv / (1.f + expf(-gv));
      }
      static_cast<T*>(p.out)[t * p.ldo + (size_t)h * vdim + i] = from_f32<T>(y);
    }
  }
}

// Local end states -> start states, in place: one thread per state element walks its request's
// segments in order.  Segment 0 starts from the request's stored state (zero for a request that
// starts); S_(p+1) = D_p S_p + L_p with D_p the product of segment p's decays (per head: the
// decay multiplied seg_len times, as the scan itself does).
template <bool PER_CHANNEL>
__global__ void linear_attention_combine_kernel(ScanParams p) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int n = p.cu_q[b + 1] - p.cu_q[b];
  const int segments = (n + p.seg_len - 1) / p.seg_len;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (segments <= 0 || e >= DIM * p.vdim) return;
  const int row = e / p.vdim;
  float s = p.fresh[b] ? 0.f : p.state[((size_t)p.state_slots[b] * p.H + h) * DIM * p.vdim + e];
  float head_decay = 1.f;
  if (!PER_CHANNEL) {
    const float d = p.decay[h];
    for (int i = 0; i < p.seg_len; ++i) head_decay *= d;
  }
  const size_t first = ((size_t)b * p.H + h) * p.max_segments;
  for (int seg = 0; seg < segments; ++seg) {
    float* at = p.seg_state + (first + seg) * DIM * p.vdim + e;
    const float local = seg + 1 < segments ? *at : 0.f;
    *at = s;
    const float d = PER_CHANNEL ? (seg + 1 < segments ? p.seg_decay[(first + seg) * DIM + row] : 0.f) : head_decay;
    s = fmaf(d, s, local);
  }
}

template <typename T, bool PER_CHANNEL, int MODE>
int launch_scan_mode(const ScanParams& p, int num_requests, int segments, cudaStream_t stream) {
  const int threads = (p.cols * GROUPS + 31) / 32 * 32;
  const size_t smem = ((size_t)(PER_CHANNEL ? 3 : 2) * CHUNK * GROUPS * RP + 2 * (size_t)CHUNK * p.cols) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(linear_attention_scan_kernel<T, PER_CHANNEL, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("linear_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  TS_LAUNCH("linear_attention", (linear_attention_scan_kernel<T, PER_CHANNEL, MODE>),
            dim3(num_requests * p.col_tiles, p.H, segments), threads, smem, stream, p);
  return 0;
}

template <typename T, bool PER_CHANNEL>
int launch_scan(const ScanParams& p, int num_requests, int num_tokens, cudaStream_t stream) {
  if (p.seg_len <= 0) {
    if (int rc = launch_scan_mode<T, PER_CHANNEL, SCAN_WHOLE>(p, num_requests, 1, stream)) return rc;
  } else {
    if (int rc = launch_scan_mode<T, PER_CHANNEL, SCAN_LOCAL>(p, num_requests, p.max_segments, stream)) return rc;
    const int elements = DIM * p.vdim;
    TS_LAUNCH("linear_attention_combine", linear_attention_combine_kernel<PER_CHANNEL>,
              dim3(num_requests, p.H, (elements + 255) / 256), 256, 0, stream, p);
    if (int rc = launch_scan_mode<T, PER_CHANNEL, SCAN_FROM_SEGMENT>(p, num_requests, p.max_segments, stream)) return rc;
  }
  if (p.raw_out)
    TS_LAUNCH("linear_attention_finish", linear_attention_finish_kernel<T>, num_tokens, p.H >= 8 ? 256 : 128, 0, stream, p,
              num_tokens);
  return 0;
}

}  // namespace

TS_EXPORT int ts_linear_attention_key_dim() { return DIM; }

TS_EXPORT int ts_linear_attention(int dtype, const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                  long long ldv, const void* gate, long long ldg, const float* z, long long ldz,
                                  float tau, const float* decay, const int* positions, const float* cos,
                                  const float* sin, int rotary_dim, float q_scale, float k_scale, float* state,
                                  const int* state_slots, const int* fresh, const int* cu_q, int num_requests,
                                  const void* norm_weight, int norm_weight_is_f32, float eps, void* out, long long ldo,
                                  int H, int vdim, int seg_len, float* seg_state, float* seg_decay, int max_segments,
                                  int num_tokens, float* raw_out, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && H > 0 && vdim > 0, "linear_attention: empty input");
  const int cols = vdim < MAX_THREADS / GROUPS ? vdim : MAX_THREADS / GROUPS;
  const int col_tiles = (vdim + cols - 1) / cols;
  TS_REQUIRE((col_tiles > 1) == (raw_out != nullptr) && num_tokens > 0,
             "linear_attention: heads of more than %d value columns come with a 32-bit scratch for their outputs, others without",
             MAX_THREADS / GROUPS);
  TS_REQUIRE((z != nullptr) != (decay != nullptr), "linear_attention: either per-channel logits or per-head decays");
  TS_REQUIRE(z == nullptr || tau > 0.f, "linear_attention: tau must be positive");
  TS_REQUIRE(rotary_dim >= 0 && rotary_dim <= DIM && rotary_dim % 2 == 0, "linear_attention: rotary_dim %d does not fit key size %d", rotary_dim, DIM);
  TS_REQUIRE(rotary_dim == 0 || (cos && sin && positions), "linear_attention: rotary without tables");
  TS_REQUIRE(q && k && v && out && state && state_slots && fresh && cu_q, "linear_attention: a null operand");
  TS_REQUIRE(seg_len == 0 || (seg_len % CHUNK == 0 && seg_state && max_segments > 0 && max_segments <= 65535 &&
                              (z == nullptr || seg_decay)),
             "linear_attention: segments of a multiple of %d tokens with scratch for their states", CHUNK);
  ScanParams p{q, k, v, gate, ldq, ldk, ldv, ldg, z, ldz, decay, z ? 1.f / tau : 0.f, positions, cos, sin, rotary_dim,
               q_scale, k_scale, state, state_slots, fresh, cu_q, norm_weight, norm_weight_is_f32, eps, out, ldo, H, vdim,
               seg_len, seg_state, seg_decay, max_segments, cols, col_tiles, raw_out};
  if (dtype == TS_F32)
    return z ? launch_scan<float, true>(p, num_requests, num_tokens, stream) : launch_scan<float, false>(p, num_requests, num_tokens, stream);
  if (dtype == TS_BF16)
    return z ? launch_scan<__nv_bfloat16, true>(p, num_requests, num_tokens, stream)
             : launch_scan<__nv_bfloat16, false>(p, num_requests, num_tokens, stream);
  return ts_fail("linear_attention: unknown dtype %d", dtype);
}
