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
// decoded token and a prompt portion of any length alike.  Thread (column c, row group g) keeps
// rows [g R, (g + 1) R) of column c of the state in registers (R = key size / 4); the four
// groups of a column are neighbouring lanes and add their shares of o_t by shuffles.  Tokens
// are staged through shared memory sixteen at a time (rotary, factors and decays applied while
// staging), and the output norm and gate run once per sixteen tokens on the staged outputs.
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
};

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, bool PER_CHANNEL>
__global__ void linear_attention_scan_kernel(ScanParams p) {
  extern __shared__ float smem[];
  const int vdim = p.vdim;
  float* sq = smem;                                   // [CHUNK][GROUPS][RP]
  float* sk = sq + CHUNK * GROUPS * RP;
  float* sa = sk + CHUNK * GROUPS * RP;               // PER_CHANNEL only
  float* sv = sa + (PER_CHANNEL ? CHUNK * GROUPS * RP : 0);   // [CHUNK][vdim]
  float* so = sv + CHUNK * vdim;                      // [CHUNK][vdim]
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int t0 = p.cu_q[b], t1 = p.cu_q[b + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, c = tid / GROUPS, g = tid % GROUPS;
  const bool owner = c < vdim;
  const int slot = p.state_slots[b];
  float* S = p.state + (((size_t)slot * p.H + h) * DIM + (size_t)g * R) * vdim + c;
  float s[R];
  if (owner && !p.fresh[b]) {
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = S[(size_t)r * vdim];
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
      sq[where] = qa * p.q_scale;
      sk[where] = ka * p.k_scale;
      if (PER_CHANNEL) sa[where] = expf(log_sigmoid(p.z[t * p.ldz + (size_t)h * DIM + i]) * p.inv_tau);
    }
    for (int idx = tid; idx < n * vdim; idx += blockDim.x) {
      const int tok = idx / vdim, i = idx % vdim;
      sv[tok * vdim + i] = to_f32<T>(v[(size_t)(base + tok) * p.ldv + i]);
    }
    __syncthreads();
    {       // (threads beyond the columns run along with a value of zero: the shuffles need whole warps)
      for (int tok = 0; tok < n; ++tok) {
        const float* qr = sq + (tok * GROUPS + g) * RP;
        const float* kr = sk + (tok * GROUPS + g) * RP;
        const float* ar = sa + (tok * GROUPS + g) * RP;
        const float vv = owner ? sv[tok * vdim + c] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float a = PER_CHANNEL ? ar[r] : head_decay;
          s[r] = fmaf(a, s[r], kr[r] * vv);
          acc = fmaf(s[r], qr[r], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (g == 0 && owner) so[tok * vdim + c] = acc;
      }
    }
    __syncthreads();
    // output norm over the value size, gate, store: a warp per token
    for (int tok = warp; tok < n; tok += warps) {
      const size_t t = base + tok;
      float acc = 0.f;
      for (int i = lane; i < vdim; i += 32) acc += so[tok * vdim + i] * so[tok * vdim + i];
      const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + p.eps);
      for (int i = lane; i < vdim; i += 32) {
        float o = so[tok * vdim + i] * rstd;
        if (p.norm_weight) o *= nw[i];
        if (p.gate) {
          const float gv = to_f32<T>(gate[t * p.ldg + i]);
          o *= gv / (1.f + expf(-gv));
        }
        out[t * p.ldo + i] = from_f32<T>(o);
      }
    }
    __syncthreads();
  }
  if (owner) {
#pragma unroll
    for (int r = 0; r < R; ++r) S[(size_t)r * vdim] = s[r];
  }
}

template <typename T, bool PER_CHANNEL>
int launch_scan(const ScanParams& p, int num_requests, cudaStream_t stream) {
  const int threads = (p.vdim * GROUPS + 31) / 32 * 32;
  const size_t smem = ((size_t)(PER_CHANNEL ? 3 : 2) * CHUNK * GROUPS * RP + 2 * (size_t)CHUNK * p.vdim) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(linear_attention_scan_kernel<T, PER_CHANNEL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("linear_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  TS_LAUNCH("linear_attention", (linear_attention_scan_kernel<T, PER_CHANNEL>), dim3(num_requests, p.H), threads, smem,
            stream, p);
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
                                  int H, int vdim, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && H > 0 && vdim > 0, "linear_attention: empty input");
  TS_REQUIRE(vdim * GROUPS <= 1024, "linear_attention: value size %d is above %d", vdim, 1024 / GROUPS);
  TS_REQUIRE((z != nullptr) != (decay != nullptr), "linear_attention: either per-channel logits or per-head decays");
  TS_REQUIRE(z == nullptr || tau > 0.f, "linear_attention: tau must be positive");
  TS_REQUIRE(rotary_dim >= 0 && rotary_dim <= DIM && rotary_dim % 2 == 0, "linear_attention: rotary_dim %d does not fit key size %d", rotary_dim, DIM);
  TS_REQUIRE(rotary_dim == 0 || (cos && sin && positions), "linear_attention: rotary without tables");
  TS_REQUIRE(q && k && v && out && state && state_slots && fresh && cu_q, "linear_attention: a null operand");
  ScanParams p{q, k, v, gate, ldq, ldk, ldv, ldg, z, ldz, decay, z ? 1.f / tau : 0.f, positions, cos, sin, rotary_dim,
               q_scale, k_scale, state, state_slots, fresh, cu_q, norm_weight, norm_weight_is_f32, eps, out, ldo, H, vdim};
  if (dtype == TS_F32) return z ? launch_scan<float, true>(p, num_requests, stream) : launch_scan<float, false>(p, num_requests, stream);
  if (dtype == TS_BF16)
    return z ? launch_scan<__nv_bfloat16, true>(p, num_requests, stream) : launch_scan<__nv_bfloat16, false>(p, num_requests, stream);
  return ts_fail("linear_attention: unknown dtype %d", dtype);
}
