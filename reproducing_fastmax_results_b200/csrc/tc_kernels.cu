// tcgen05 / TMEM kernels of the Fastmax engine: bf16 operands, fp32 accumulation in tensor memory; head dim 64,
// order 1 and 2, with and without a mask, carried moment states in and out.  The 2369 feature rows of the order-2
// state are cut into 19 tiles of 128 rows (18 tiles of two 8x8-block pair units + the tile with the linear and
// constant features); a scan CTA = (batch*head, slice of up to 4 tiles); order 1 is the last tile alone.
// This file holds what the scans share and the host side:
//   Sched              which chunks of a scan apply the state / update it / refresh its bf16 copy
//   intra_fwd_kernel   O'_c += tril f(Q_c K_c^T) [V_c | 1], one CTA per (chunk, head), parallel over chunks
//   tc_bwd.cuh         intra-chunk backward kernel, dO' prologue
//   tc_scan2.cuh       forward scan and dv scan ("apply + update", Phi operands in tensor memory)
//   tc_scan3.cuh       dq and dk scans (dphi + chain rule + update)
//   tc_forward / tc_backward: scan geometry and schedules, tensor maps, workspace layout, launch sequences,
//                      segmentation of long batch-1 sequences with few heads
// Every device-side wait is bounded: on a timeout a role records an error code, raises the CTA's abort flag, and
// the CTA frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "launchers.cuh"
#include "tc_launchers.cuh"
#include "tc_ptx.cuh"

namespace fm {

__device__ int g_tc_status = 0;
// how often each wait site of the tensor-core kernels gave up first in its CTA (index = code & 255); diagnostics only
__device__ int g_tc_wait_hist[256];

namespace tc {

constexpr int CH = 128;                 // tokens per chunk
constexpr int REGION = 16384;           // 128 rows x 128 B
constexpr int TILE = 2 * REGION;        // a 128 x 128 bf16 operand tile
constexpr int BLK = 2048;               // one 8-column block of an MN-major operand: 128 rows x 16 B
constexpr int SB_TILE = 9 * BLK;        // 72 columns stored; the MMA's columns 72..79 read the bytes that follow
constexpr int NTILES = 19;
constexpr long long WAIT_CYCLES = 4000000000ll;       // ~2 s at 2 GHz

// Which chunks of a scan (by scan index ci = 0 .. nchunks-1, in the order the scan visits them) read the state and
// which ones add to it.  A chunk "applies" when some of its positions hold rows of the tile that multiplies the state
// (queries in the forward and dq scans, keys in the dk and dv scans) and the state is not trivially zero; it
// "updates" when some of its positions hold rows that build the state and a later chunk (or the caller, through
// state_out) still needs the result.  Both sets are contiguous ranges; a range with first > last is empty.  The
// bf16 copy of the state is refreshed after the updates c_first .. c_last, i.e. only where an apply follows before the
// next update (and once before chunk 0 when the state starts from a caller-provided array, h = 1).  Every role of a scan kernel derives its barrier phase counts from
// these ranges, so causal calls with nk > nq, calls with a carried state and the non-causal layout (all keys first,
// then all queries) run through the same code.
// Phase discipline: an mbarrier wait names a phase by its parity only, so a waiter must see every completion of a
// barrier it uses, in order, and may never fall two completions behind.  That is why the update issuer signals
// "S_t is final" (S_DONE) only for the chunks somebody waits on (the copies, and the last update when the caller
// wants the final state, s_final = 1) instead of for every update, and why the host declines layouts in which a
// carried state meets update-only chunks before the first apply.
struct Sched {
  int a_first, a_last;
  int u_first, u_last;
  int c_first, c_last;
  int h;
  int s_final;
  __host__ __device__ static int clampi(int x, int lo, int hi) { return x < lo ? lo : (x > hi ? hi : x); }
  __host__ __device__ bool A(int ci) const { return ci >= a_first && ci <= a_last; }
  __host__ __device__ bool U(int ci) const { return ci >= u_first && ci <= u_last; }
  __host__ __device__ bool C(int ci) const { return ci >= c_first && ci <= c_last; }
  __host__ __device__ int na_total() const { return a_last >= a_first ? a_last - a_first + 1 : 0; }
  __host__ __device__ int nu_total() const { return u_last >= u_first ? u_last - u_first + 1 : 0; }
  __host__ __device__ int na_before(int ci) const { return clampi(ci - a_first, 0, na_total()); }   // applies in chunks < ci
  __host__ __device__ int nu_before(int ci) const { return clampi(ci - u_first, 0, nu_total()); }   // updates in chunks < ci
  __host__ __device__ int ncv_total() const { return c_last >= c_first ? c_last - c_first + 1 : 0; }
  __host__ __device__ bool SD(int ci) const { return C(ci) || (s_final && ci == u_last); }        // update ci signals S_DONE
  __host__ __device__ int nc_before(int ci) const {                                                 // copies made before chunk ci
    return h + clampi(ci - c_first, 0, c_last >= c_first ? c_last - c_first + 1 : 0);
  }
};

struct FwdParams {
  float* oacc;   // [BH][nq][68]
  int heads, nq, nk, off, nchunks;
  float c0, c1, c2;
};

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ float tile_weight(int gt, int f, float c0, float c1, float c2) {
  if (gt < NTILES - 1) {
    int a, b;
    pair_decode(2 * gt + (f >> 6), 8, a, b);
    return (a == b) ? c2 : 2.f * c2;
  }
  return f < 64 ? c1 : (f == 64 ? c0 : 0.f);
}

// 8 fp32 values (as raw bits) * w -> 8 bf16 -> one 16-byte store
__device__ __forceinline__ void store_block8(uint8_t* dst, const uint32_t* r, float w) {
  uint4 o;
  o.x = pack_bf16(__uint_as_float(r[0]) * w, __uint_as_float(r[1]) * w);
  o.y = pack_bf16(__uint_as_float(r[2]) * w, __uint_as_float(r[3]) * w);
  o.z = pack_bf16(__uint_as_float(r[4]) * w, __uint_as_float(r[5]) * w);
  o.w = pack_bf16(__uint_as_float(r[6]) * w, __uint_as_float(r[7]) * w);
  *reinterpret_cast<uint4*>(dst) = o;
}
// 8 fp32 values (as raw bits) -> 8 bf16 -> one 16-byte store
__device__ __forceinline__ void store_block8_plain(uint8_t* dst, const uint32_t* r) {
  uint4 o;
  o.x = pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1]));
  o.y = pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3]));
  o.z = pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5]));
  o.w = pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7]));
  *reinterpret_cast<uint4*>(dst) = o;
}


// ------------------------------------------------------------------------------------------------------
// intra-chunk causal term, one CTA per (chunk, batch*head):  O'_c += tril(f(Q_c K_c^T)) [V_c | 1]
// ------------------------------------------------------------------------------------------------------
constexpr int I_THREADS = 256;
constexpr int I_OFF_Q = 0, I_OFF_K = REGION, I_OFF_VP = 2 * REGION, I_OFF_P = 2 * REGION + 9 * BLK + 2 * 1024;  // 53248
constexpr int I_OFF_BAR = I_OFF_P + TILE;
constexpr int I_SMEM_BYTES = I_OFF_BAR + 64 + 1024;
static_assert(I_OFF_P % 1024 == 0, "operand tiles with the 128-byte swizzle need 1024-byte alignment");
static_assert(CH * 68 * 4 <= I_OFF_BAR, "the output staging rows reuse the operand tiles");

__global__ void __launch_bounds__(I_THREADS, 2)
intra_fwd_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                 const __grid_constant__ CUtensorMap tmv, const FwdParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* rawq = sm + I_OFF_Q;
  uint8_t* rawk = sm + I_OFF_K;
  uint8_t* vp = sm + I_OFF_VP;
  uint8_t* pt = sm + I_OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + I_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + I_OFF_BAR + 32);

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int h = w >> 2, quarter = w & 3, l = quarter * 32 + lane;
  const int c = blockIdx.x, head = blockIdx.z;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int pos0 = c * CH;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    fence_mbar_init();
  }
  if (w == 0) tmem_alloc(tmem_slot, 256);
  if (tid < CH) *reinterpret_cast<uint4*>(vp + 8 * BLK + tid * 16) = make_uint4((pos0 + tid < P.nk) ? 0x00003F80u : 0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
  if (tid == 0) {
    mbar_arrive_expect_tx(&bars[0], 2 * REGION + 8 * BLK);
    tma_load_4d(rawq, &tmq, &bars[0], 0, pos0 - P.off, h_idx, b_idx);
    tma_load_4d(rawk, &tmk, &bars[0], 0, pos0, h_idx, b_idx);
#pragma unroll
    for (int i = 0; i < 8; ++i) tma_load_4d(vp + i * BLK, &tmv, &bars[0], 8 * i, pos0, h_idx, b_idx);
  }
  bool ok = mbar_wait_bounded(&bars[0], 0, WAIT_CYCLES);
  ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      const uint64_t dq = make_smem_desc(smem_u32(rawq), 16, 1024, 2);
      const uint64_t dk = make_smem_desc(smem_u32(rawk), 16, 1024, 2);
      constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) mma_ss(tmem_base, dq + (uint64_t)(2 * ks), dk + (uint64_t)(2 * ks), IDESC_QK, ks > 0);
      mma_commit(&bars[1]);
    }
    ok = mbar_wait_bounded(&bars[1], 0, WAIT_CYCLES);
    ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  }
  if (ok) {
    tc_fence_after_sync();
    uint8_t* region = pt + h * REGION;
    const int sw = l & 7;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t r[32];
      tmem_ld32(lane_addr + 64u * h + 32u * half, r);
      tmem_ld_wait();
#pragma unroll
      for (int jb = 0; jb < 4; ++jb) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = 64 * h + 32 * half + 8 * jb + e;
          const float s = __uint_as_float(r[8 * jb + e]);
          pv[e] = (j <= l) ? (P.c0 + s * (P.c1 + P.c2 * s)) : 0.f;
        }
        uint4 o;
        o.x = pack_bf16(pv[0], pv[1]);
        o.y = pack_bf16(pv[2], pv[3]);
        o.z = pack_bf16(pv[4], pv[5]);
        o.w = pack_bf16(pv[6], pv[7]);
        *reinterpret_cast<uint4*>(region + l * 128 + (((4 * half + jb) ^ sw) << 4)) = o;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t IDESC_PV = make_idesc_bf16(128, 80, 0, 1);
      const uint64_t dp = make_smem_desc(smem_u32(pt), 16, 1024, 2);
      const uint64_t dv = make_smem_desc(smem_u32(vp), 128, 2048, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        mma_ss(tmem_base + 128u, dp + (uint64_t)(((ks >> 2) * REGION + (ks & 3) * 32) >> 4), dv + (uint64_t)(16 * ks), IDESC_PV,
               ks > 0);
      mma_commit(&bars[1]);
    }
    ok = mbar_wait_bounded(&bars[1], 1, WAIT_CYCLES);
    ok = (__syncthreads_or(ok ? 0 : 1) == 0);
  }
  if (ok) {
    // O'_c of this chunk -> staging rows (68 floats; the operand tiles are dead by now) -> one bulk reduce-add
    tc_fence_after_sync();
    float* stage = reinterpret_cast<float*>(sm);
    float4* rowp = reinterpret_cast<float4*>(stage + l * 68 + 32 * h);
    uint32_t r[32];
    tmem_ld32(lane_addr + 128u + 32u * h, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      rowp[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                            __uint_as_float(r[4 * j + 3]));
    if (h == 0) {
      uint32_t r8[8];
      tmem_ld8(lane_addr + 128u + 64u, r8);
      tmem_ld_wait();
      reinterpret_cast<float4*>(stage + l * 68 + 64)[0] = make_float4(__uint_as_float(r8[0]), 0.f, 0.f, 0.f);
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      const long long q0 = (long long)pos0 - P.off;  // query row of staging row 0
      const int r0 = q0 < 0 ? (int)(-q0 < CH ? -q0 : CH) : 0;
      const long long lim = (long long)P.nq - q0;
      const int r1 = lim < CH ? (lim < 0 ? 0 : (int)lim) : CH;
      if (r1 > r0) {
        bulk_reduce_add_f32(P.oacc + ((long long)head * P.nq + q0 + r0) * 68, stage + r0 * 68, (uint32_t)(r1 - r0) * 272u);
        bulk_commit_group();
        bulk_wait_read_all();   // the staging rows stay valid until the copy engine has read them
      }
    }
  } else if (tid == 0) {
    atomicExch(&g_tc_status, 50);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 256);
}

#include "tc_bwd.cuh"
#include "tc_scan2.cuh"
#include "tc_scan3.cuh"
#include "tc_p1.cuh"

// Exclusive running sum over the segments of the states st[seg][head][n] (in place): forward order (prefix) or
// reverse (suffix), starting from init[head][n] when given; total_out[head][n] (optional) = init + all segments.
__global__ void seg_state_scan_kernel(float* __restrict__ st, int nseg, int heads, long long n, const float* __restrict__ init,
                                      float* __restrict__ total_out, int reverse) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // over heads * n
  if (idx >= (long long)heads * n) return;
  float run = init ? init[idx] : 0.f;
  for (int i = 0; i < nseg; ++i) {
    const int sgi = reverse ? nseg - 1 - i : i;
    float* p = st + (long long)sgi * heads * n + idx;
    const float t = *p;
    *p = run;
    run += t;
  }
  if (total_out) total_out[idx] = run;
}

// Test-only kernel for the bounded-wait failure path: one thread waits, with a limit of `cycles` SM clocks, on an
// mbarrier that nobody ever arrives on, then records wait site `code` exactly as a production role would
// (s2::fail_record: histogram, abort flag, status word) and returns normally.  No TMA, MMA or TMEM is involved.
__global__ void wait_selftest_kernel(long long cycles, int code) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_abortable(&bar, 0u, cycles, &abort_flag)) s2::fail_record(code, &abort_flag);
}

}  // namespace tc

// ------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  // function-local static with an initialiser: thread-safe, so two host threads making their first call together
  // both see the resolved entry point
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(p);
    return (EncodeTiledFn) nullptr;
  }();
  return fn;
}

// bf16 (batch, head, token, cols) view -> 4-D tensor map with a [box_rows x box_cols] box.
static bool make_map(CUtensorMap* m, const fastmax_tensor& t, int batch, int heads, int n, int box_cols, int box_rows,
                     bool swizzle128, int cols = 64) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || n <= 0) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)n, (cuuint64_t)heads, (cuuint64_t)batch};
  // a stride of a size-1 dimension is never used for addressing; any legal value will do
  cuuint64_t sn = (cuuint64_t)t.stride_n * 2, sh = (cuuint64_t)t.stride_h * 2, sbb = (cuuint64_t)t.stride_b * 2;
  if (n == 1 || sn == 0) sn = 128;
  if (heads == 1 || sh == 0) sh = sn * (cuuint64_t)n;
  if (batch == 1 || sbb == 0) sbb = 128;
  const cuuint64_t strides[3] = {sn, sh, sbb};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 || strides[i] >= (1ull << 40)) return false;
  const cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Transposed bf16 copy xt [batch*heads][64][ntp] -> 3-D tensor map (tokens, 64 dims, batch*heads), box 72 x 64, no swizzle.
static bool make_map_t(CUtensorMap* m, void* xt, int bh, int n, int ntp) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || n <= 0) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)n, 64, (cuuint64_t)bh};
  const cuuint64_t strides[2] = {(cuuint64_t)ntp * 2, (cuuint64_t)ntp * 128};
  const cuuint32_t box[3] = {72, 64, 1};  // 64 tokens + 8: shared-memory rows of 144 bytes spread over the banks
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, xt, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
static inline int tokens_padded(int n) { return (n + 63) / 64 * 64; }
static inline size_t transposed_bytes(int bh, int n) { return ((size_t)bh * 64 * tokens_padded(n) * 2 + 255) / 256 * 256; }

// xt [batch*heads][64][tokens_padded(n + shift)]: column p = token p - shift of x
static cudaError_t launch_transpose(const fastmax_tensor& x, int batch, int heads, int n, int shift, __nv_bfloat16* xt,
                                    cudaStream_t st) {
  LaunchScope ls(KK_TC_TRANSPOSE, st);
  const int ntp = tokens_padded(n + shift);
  tc::s2::transpose_tokens_kernel<<<dim3(ntp / 64, batch * heads), 256, 0, st>>>(
      View{x.ptr, x.stride_b, x.stride_h, x.stride_n}, xt, n, ntp, heads, shift);
  return cudaGetLastError();
}

// Side streams for kernels of one call that are independent of each other (each scan fills 4.3 waves of the 148
// SMs; side by side their last waves overlap).  Created once per device, on first use; forked from the caller's
// stream with an event and joined back into it, so the call as a whole is still ordered on the caller's stream.
struct SideStreams {
  std::mutex use;   // held by a call from its fork to its join: the events and streams below are shared per device
  cudaStream_t s[3] = {nullptr, nullptr, nullptr};
  cudaEvent_t fork = nullptr, mid = nullptr, aux = nullptr, join[3] = {nullptr, nullptr, nullptr};
  bool ok = false;
};
static SideStreams* side_streams() {
  static std::mutex mu;
  static SideStreams pool[64];
  static bool tried[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  SideStreams& p = pool[dev];
  if (!tried[dev]) {
    tried[dev] = true;
    bool good = cudaEventCreateWithFlags(&p.fork, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&p.mid, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&p.aux, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 3 && good; ++i)
      good = cudaStreamCreateWithFlags(&p.s[i], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&p.join[i], cudaEventDisableTiming) == cudaSuccess;
    p.ok = good;
  }
  return p.ok ? &p : nullptr;
}
// Streams for `n` independent kernels: out[0] is the caller's stream; out[1..] are side streams that wait for
// everything enqueued on the caller's stream so far (or the caller's stream itself when side streams are off).
// `lock` keeps the device's side streams for this call until it goes out of scope in the caller (after the join has
// been enqueued): a stream wait takes the event's record of that moment, so two host threads interleaving their
// record / wait pairs on the shared events would order their kernels wrongly.
static SideStreams* fork_streams(const fastmax_problem* pb, cudaStream_t st, int n, cudaStream_t* out,
                                 std::unique_lock<std::mutex>& lock) {
  for (int i = 0; i < n; ++i) out[i] = st;
  if ((pb->flags & FASTMAX_FLAG_SINGLE_STREAM) || profiling_on()) return nullptr;
  SideStreams* p = side_streams();
  if (!p) return nullptr;
  lock = std::unique_lock<std::mutex>(p->use);
  if (cudaEventRecord(p->fork, st) != cudaSuccess) return nullptr;
  for (int i = 1; i < n; ++i) {
    if (cudaStreamWaitEvent(p->s[i - 1], p->fork, 0) != cudaSuccess) return nullptr;
    out[i] = p->s[i - 1];
  }
  return p;
}
static cudaError_t join_streams(SideStreams* p, cudaStream_t st, int n) {
  if (!p) return cudaSuccess;
  for (int i = 1; i < n; ++i) {
    cudaError_t e = cudaEventRecord(p->join[i - 1], p->s[i - 1]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st, p->join[i - 1], 0);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (device, kernel) instead of on every call: the attribute
// sticks to the function on that device.  `slot` numbers the kernels of this file.
template <typename K>
static cudaError_t ensure_smem(K kernel, int bytes, int slot) {
  static std::mutex mu;
  static bool done[64][8] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || slot < 0 || slot >= 8) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  std::lock_guard<std::mutex> lk(mu);
  if (done[dev][slot]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[dev][slot] = true;
  return e;
}

// Joins the side streams back into the caller's stream when a call leaves between its fork and its join (an error
// return): the side streams must never be left holding work the caller's stream does not wait for.
struct JoinOnExit {
  SideStreams* p;
  cudaStream_t st;
  int n;
  bool joined = false;
  ~JoinOnExit() {
    if (!joined) join_streams(p, st, n);
  }
};

// Positions of a call: keys sit at positions 0 .. nk-1.  Causal: query l sits at position nk - nq + l (it sees the keys
// up to its own position).  Non-causal: the queries follow the keys, from the next chunk boundary on, so every query
// sees every key and no chunk holds both; the intra-chunk (masked) kernels are then not needed at all.
struct ScanGeom {
  int k0;            // position of query 0
  int nch;           // chunks of 128 positions
  int qc0, qc1;      // chunks that hold queries
  int kc0, kc1;      // chunks that hold keys
  int nslices, tps, tile_first, state_rows;
};
static int device_sms();
static ScanGeom scan_geom(const fastmax_problem* pb, bool backward = false) {
  ScanGeom g{};
  g.k0 = pb->causal ? pb->nk - pb->nq : (pb->nk + tc::CH - 1) / tc::CH * tc::CH;
  const int npos = pb->causal ? pb->nk : g.k0 + pb->nq;
  g.nch = (npos + tc::CH - 1) / tc::CH;
  g.qc0 = g.k0 / tc::CH;
  g.qc1 = pb->nq > 0 ? (g.k0 + pb->nq - 1) / tc::CH : g.qc0 - 1;
  g.kc0 = 0;
  g.kc1 = (pb->nk - 1) / tc::CH;
  // Order 2: 19 feature tiles per head, four per thread block (5 slices) or three (7 slices: more, shorter blocks; a
  // block of three tiles takes 0.79 of the time of one of four, so four are 5 % more efficient per tile).  What decides
  // is how many whole rounds of blocks the 148 SMs run: one scan kernel at a time in the forward call, the three scans
  // of the backward call side by side.  Three tiles are taken where they save a round.  Measured on B x H16 x N4096,
  // forward alone / whole step: 16 heads 0.110 vs 0.127 ms with three tiles in the forward call and 0.446 vs 0.459 ms
  // with four in the backward call; 32 heads 0.200 vs 0.225 and 0.785 vs 0.835; 48 heads and from 96 up four tiles in
  // both (128 heads: 0.52 vs 0.54 ms forward scan).
  g.tps = 4;
  if (pb->order == 2) {
    const long long bh = (long long)pb->batch * pb->heads, sms = device_sms(), kernels = backward ? 3 : 1;
    const long long rounds4 = (kernels * 5 * bh + sms - 1) / sms, rounds3 = (kernels * 7 * bh + sms - 1) / sms;
    // the backward's three scans differ in length, so its rounds are only roughly whole: a wider margin there
    if ((double)rounds3 * 0.786 < (backward ? 0.90 : 0.97) * (double)rounds4) g.tps = 3;
  }
  g.nslices = pb->order == 2 ? (tc::NTILES + g.tps - 1) / g.tps : 1;
  g.tile_first = pb->order == 2 ? 0 : tc::NTILES - 1;
  g.state_rows = pb->order == 2 ? 64 * 36 + 65 : 65;
  return g;
}
// Schedule of one scan.  Forward direction (forward pass, dq): query chunks apply, key chunks update.  Reverse
// direction (dk, dv): key chunks apply, query chunks update, and scan index ci visits chunk nch - 1 - ci.
static tc::Sched make_sched(const ScanGeom& g, bool reverse, bool has_init, bool want_apply, bool want_state) {
  tc::Sched sc{};
  int a0, a1, u0, u1;
  if (!reverse) { a0 = g.qc0; a1 = g.qc1; u0 = g.kc0; u1 = g.kc1; }
  else { a0 = g.nch - 1 - g.kc1; a1 = g.nch - 1 - g.kc0; u0 = g.nch - 1 - g.qc1; u1 = g.nch - 1 - g.qc0; }
  if (!want_apply) { a0 = 0; a1 = -1; }
  else if (!has_init && a0 == 0) a0 = 1;           // the state is still zero in the first chunk
  if (!want_state && u1 > a1 - 1) u1 = a1 - 1;     // updates that nothing reads any more
  sc.a_first = a0; sc.a_last = a1; sc.u_first = u0; sc.u_last = u1;
  sc.c_first = u0 > a0 - 1 ? u0 : a0 - 1;
  sc.c_last = u1 < a1 - 1 ? u1 : a1 - 1;
  sc.h = has_init ? 1 : 0;
  sc.s_final = (want_state && sc.nu_total() > 0 && !sc.C(u1)) ? 1 : 0;
  return sc;
}

static bool tc_kernels_cover(const fastmax_problem* pb) {
  if (pb->flags & FASTMAX_FLAG_NO_TENSOR_CORES) return false;
  if (pb->dtype != FASTMAX_BF16 || pb->d != 64 || (pb->order != 1 && pb->order != 2)) return false;
  if (pb->nk <= 0) return false;
  if ((long long)pb->nk + pb->nq + 2 * tc::CH >= (1ll << 30)) return false;
  return true;
}
static bool tc_enough_blocks(const fastmax_problem* pb) {
  return (long long)pb->batch * pb->heads * (pb->order == 2 ? 5 : 1) >= 64;   // one scan CTA per (head, slice)
}
static bool tc_common_supported(const fastmax_problem* pb) { return tc_kernels_cover(pb) && tc_enough_blocks(pb); }

// Long causal sequences with few heads (one scan CTA per (head, slice) would leave most SMs idle): the sequence of a
// batch-1 call is cut into `nseg` segments that the kernels see as the batch dimension (segment s of every tensor
// is the view starting at token s * L, so nothing is copied).  Three steps, all on the tensor-memory kernels:
// (1) the moment state of every segment's keys (update-only scans), (2) an exclusive prefix over the segments,
// (3) the ordinary call on the segment view with the prefixes as carried states.  The backward does the same for
// the gradient moments with an exclusive suffix.  Returns the number of segments, or 0 when the call does not
// qualify (then the CUDA-core engine, which segments on its own, takes it).
static int tc_segments(const fastmax_problem* pb) {
  if (!tc_kernels_cover(pb) || tc_enough_blocks(pb)) return 0;
  if (!pb->causal || pb->batch != 1 || pb->nq != pb->nk || pb->nq < 4 * tc::CH) return 0;
  const long long per_seg = (long long)pb->heads * (pb->order == 2 ? 5 : 1);
  int nseg = 2;
  while (per_seg * nseg < 2ll * device_sms() && nseg < 4096) nseg *= 2;     // about two waves of scan CTAs
  while (nseg > 1 && (pb->nq % (nseg * tc::CH) != 0 || pb->nq / nseg < 2 * tc::CH)) nseg /= 2;
  if (nseg < 2 || per_seg * nseg < 64) return 0;
  return nseg;
}
static fastmax_tensor seg_view(const fastmax_tensor& t, int seg_len) {
  fastmax_tensor v = t;
  v.stride_b = (int64_t)seg_len * t.stride_n;
  return v;
}
static fastmax_problem seg_problem(const fastmax_problem* pb, int nseg) {
  fastmax_problem vp = *pb;
  vp.batch = nseg;
  vp.nq = vp.nk = pb->nq / nseg;
  return vp;
}
static size_t seg_state_bytes(const fastmax_problem* pb, int nseg) {
  const size_t rows = pb->order == 2 ? 64 * 36 + 65 : 65;
  return ((size_t)nseg * pb->heads * rows * 68 * sizeof(float) + 255) / 256 * 256;
}

// ---- bf16 with a head dim below 64 -----------------------------------------------------------------------------------
// The kernels are built for 64-wide heads.  A narrower bf16 head is zero-padded to 64 columns in the workspace: the
// added dimensions contribute nothing to any score, moment, output or gradient, so the results are those of the
// narrow problem.  Four times the arithmetic a 32-wide head strictly needs, on an engine that is about twenty times
// faster per operation than the CUDA cores.  Carried states are converted between the 32-wide and the 64-wide layout
// on the way in and out (state_width_kernel).
namespace tc {
// x: strided [batch][heads][n][d] bf16 view, out: dense [batch*heads][n][64]; a thread moves eight columns
__global__ void pad_cols_kernel(View x, int d, int n, int heads, uint4* __restrict__ out, long long nrows) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = idx >> 3;
  const int c8 = (int)(idx & 7);
  if (row >= nrows) return;
  const int l = (int)(row % n);
  const int head = (int)(row / n), b = head / heads, h = head - b * heads;
  uint4 val = make_uint4(0u, 0u, 0u, 0u);
  if (c8 * 8 < d)
    val = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (long long)b * x.sb + (long long)h * x.sh +
                                          (long long)l * x.sn + c8 * 8);
  out[idx] = val;
}
// in: dense [batch*heads][n][64], y: strided view of width d
__global__ void unpad_cols_kernel(const uint4* __restrict__ in, int d, int n, int heads, View y, long long nrows) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = idx >> 3;
  const int c8 = (int)(idx & 7);
  if (row >= nrows || c8 * 8 >= d) return;
  const int l = (int)(row % n);
  const int head = (int)(row / n), b = head / heads, h = head - b * heads;
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(y.ptr)) + (long long)b * y.sb + (long long)h * y.sh +
                            (long long)l * y.sn + c8 * 8) = in[idx];
}
// Moment states between the 32-wide layout ([heads][rows32][36]: pair units of the 4 x 4 block grid, 32 linear rows, the
// constant; columns 0..31 values, 32 the denominator moment) and the 64-wide one ([heads][rows64][68], 8 x 8 grid,
// denominator in column 64).  Every row / column of the narrow state has one place in the wide one; the rest of the
// wide state belongs to the padded dimensions and is zero.  widen: scatter into a zeroed wide state; else gather.
__global__ void state_width_kernel(const float* __restrict__ src, float* __restrict__ dst, int order, int widen, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one element of the narrow state
  if (idx >= total) return;
  const int rows32 = order == 2 ? 673 : 33, rows64 = order == 2 ? 2369 : 65;
  const int c = (int)(idx % 36);
  const long long hr = idx / 36;
  const int r = (int)(hr % rows32);
  const long long head = hr / rows32;
  int r64;
  const int npair = order == 2 ? 640 : 0;
  if (r < npair) {
    int a, b;
    pair_decode(r >> 6, 4, a, b);
    r64 = 64 * (a * 8 - a * (a - 1) / 2 + (b - a)) + (r & 63);
  } else if (r < npair + 32) {
    r64 = (order == 2 ? 2304 : 0) + (r - npair);
  } else {
    r64 = rows64 - 1;
  }
  const int c64 = c < 32 ? c : (c == 32 ? 64 : -1);
  const long long wide = (head * rows64 + r64) * 68 + c64;
  if (widen) {
    if (c64 >= 0) dst[wide] = src[idx];
  } else {
    dst[idx] = c64 >= 0 ? src[wide] : 0.f;
  }
}
}  // namespace tc

static size_t wide_state_bytes(const fastmax_problem* pb) {
  return ((size_t)pb->batch * pb->heads * (pb->order == 2 ? 2369 : 65) * 68 * sizeof(float) + 255) / 256 * 256;
}
static cudaError_t launch_state_width(const float* src, float* dst, const fastmax_problem* pb, bool widen, cudaStream_t st) {
  const long long total = (long long)pb->batch * pb->heads * (pb->order == 2 ? 673 : 33) * 36;
  if (widen) {
    cudaError_t e = cudaMemsetAsync(dst, 0, wide_state_bytes(pb), st);
    if (e != cudaSuccess) return e;
  }
  LaunchScope ls(KK_TC_PAD, st);
  tc::state_width_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(src, dst, pb->order, widen ? 1 : 0, total);
  return cudaGetLastError();
}

static bool pad_view_ok(const fastmax_tensor& t) {   // 128-bit accesses on every row
  return t.ptr && ((uintptr_t)t.ptr & 15) == 0 && (t.stride_b & 7) == 0 && (t.stride_h & 7) == 0 && (t.stride_n & 7) == 0;
}
static bool tc_narrow_head(const fastmax_problem* pb) {
  // D = 16 is left to the CUDA cores: sixteen times the arithmetic makes the padded call no faster (config 2's shape:
  // 2.98 ms padded against 3.03 ms; at D = 32 it is 2.98 ms against 10.0 ms)
  return !(pb->flags & FASTMAX_FLAG_NO_TENSOR_CORES) && pb->dtype == FASTMAX_BF16 && pb->d == 32;
}
static size_t padded_bytes(const fastmax_problem* pb, int n) {
  return ((size_t)pb->batch * pb->heads * n * 64 * sizeof(__nv_bfloat16) + 255) / 256 * 256;
}
static fastmax_tensor padded_view(void* p, const fastmax_problem* pb, int n) {
  return fastmax_tensor{p, (int64_t)pb->heads * n * 64, (int64_t)n * 64, 64};
}
static cudaError_t launch_pad(const fastmax_tensor& x, const fastmax_problem* pb, int n, void* out, cudaStream_t st) {
  const long long nrows = (long long)pb->batch * pb->heads * n;
  if (nrows == 0) return cudaSuccess;
  LaunchScope ls(KK_TC_PAD, st);
  tc::pad_cols_kernel<<<(unsigned)((nrows * 8 + 255) / 256), 256, 0, st>>>(View{x.ptr, x.stride_b, x.stride_h, x.stride_n}, pb->d, n,
                                                                         pb->heads, (uint4*)out, nrows);
  return cudaGetLastError();
}
static cudaError_t launch_unpad(const void* in, const fastmax_problem* pb, int n, const fastmax_tensor& y, cudaStream_t st) {
  const long long nrows = (long long)pb->batch * pb->heads * n;
  if (nrows == 0) return cudaSuccess;
  LaunchScope ls(KK_TC_PAD, st);
  tc::unpad_cols_kernel<<<(unsigned)((nrows * 8 + 255) / 256), 256, 0, st>>>((const uint4*)in, pb->d, n, pb->heads,
                                                                           View{y.ptr, y.stride_b, y.stride_h, y.stride_n}, nrows);
  return cudaGetLastError();
}
// the 64-wide problem and arguments of a narrow forward call, over buffers at `base` (nullptr: only for the predicates);
// a state-only call (no output) has no q: the keys stand in, as they do for the caller
static void padded_forward(const fastmax_problem* pb, const fastmax_forward_args* a, char* base, fastmax_problem& pp,
                           fastmax_forward_args& in, size_t& used) {
  pp = *pb;
  pp.d = 64;
  char* const p0 = base ? base : (char*)256;   // never dereferenced when base is null
  char* p = p0;
  const bool want_o = a->o.ptr != nullptr;
  in = fastmax_forward_args{};
  in.k = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
  in.v = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
  if (want_o) {
    in.q = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
    in.o = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
    in.g = a->g;
  } else {
    in.q = in.k;
  }
  if (a->state_in) { in.state_in = (const float*)p; p += wide_state_bytes(pb); }
  if (a->state_out) { in.state_out = (float*)p; p += wide_state_bytes(pb); }
  in.key_moments_in = a->key_moments_in;     // per-segment moments of the padded problem: opaque to the caller
  in.key_moments_out = a->key_moments_out;
  used = (size_t)(p - p0);
}
static void padded_backward(const fastmax_problem* pb, const fastmax_backward_args* a, char* base, fastmax_problem& pp,
                            fastmax_backward_args& in, size_t& used) {
  pp = *pb;
  pp.d = 64;
  char* const p0 = base ? base : (char*)256;
  char* p = p0;
  in = fastmax_backward_args{};
  in.q = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
  in.k = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
  in.v = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
  in.o = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
  in.d_out = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
  if (a->dq.ptr) {
    in.dq = padded_view(p, pb, pb->nq); p += padded_bytes(pb, pb->nq);
    in.dk = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
    in.dv = padded_view(p, pb, pb->nk); p += padded_bytes(pb, pb->nk);
  }
  in.g = a->g;
  if (a->state_in) { in.state_in = (const float*)p; p += wide_state_bytes(pb); }
  if (a->dstate_in) { in.dstate_in = (const float*)p; p += wide_state_bytes(pb); }
  if (a->dstate_out) { in.dstate_out = (float*)p; p += wide_state_bytes(pb); }
  in.key_moments_in = a->key_moments_in;
  in.grad_moments_in = a->grad_moments_in;
  in.grad_moments_out = a->grad_moments_out;
  used = (size_t)(p - p0);
}
static bool tc_forward_paddable(const fastmax_problem* pb, const fastmax_forward_args* a);
static bool tc_backward_paddable(const fastmax_problem* pb, const fastmax_backward_args* a);

static bool tc_forward_supported(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (!tc_common_supported(pb)) return false;
  const bool want_o = a->o.ptr && pb->nq > 0;
  if (!want_o && !a->state_out) return false;
  if (!pb->causal && a->state_in) return false;
  if (a->state_in && pb->nk != pb->nq) return false;   // see the phase discipline note at Sched
  return true;
}

static bool tc_forward_segmentable(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (tc_segments(pb) <= 0 || !a->k.ptr || !a->v.ptr) return false;
  if (a->o.ptr) return a->q.ptr && a->g.ptr;
  return a->state_out != nullptr;   // a state-only call: the segment moments and their sum
}

size_t tc_forward_workspace(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (tc_forward_paddable(pb, a)) {
    fastmax_problem pp;
    fastmax_forward_args in;
    size_t used;
    padded_forward(pb, a, nullptr, pp, in, used);
    return used + tc_forward_workspace(&pp, &in) + 256;
  }
  if (tc_forward_segmentable(pb, a)) {
    // segment states + the workspace of the larger of the two inner calls
    const int nseg = tc_segments(pb);
    const fastmax_problem vp = seg_problem(pb, nseg);
    fastmax_forward_args mom{};   // the state-only call over the segments
    mom.q = a->k; mom.k = a->k; mom.v = a->v;
    float dummy = 0.f;
    mom.state_out = &dummy;
    size_t inner = tc_forward_workspace(&vp, &mom);
    if (a->o.ptr) {               // the full call on the segment view
      fastmax_forward_args in = *a;
      in.state_in = &dummy; in.state_out = nullptr;
      in.key_moments_in = nullptr; in.key_moments_out = nullptr;
      const size_t full = tc_forward_workspace(&vp, &in);
      if (full > inner) inner = full;
    }
    return seg_state_bytes(pb, nseg) + inner;
  }
  if (!tc_forward_supported(pb, a)) return 0;
  const bool want_o = a->o.ptr && pb->nq > 0;
  return (want_o ? ((size_t)pb->batch * pb->heads * pb->nq * 68 * sizeof(float) + 255) / 256 * 256 : 0) +
         transposed_bytes(pb->batch * pb->heads, pb->nk);
}

// Order 1 without a mask: one kernel, no workspace (tc_p1.cuh).
static bool tc_p1_supported(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (pb->flags & FASTMAX_FLAG_NO_TENSOR_CORES) return false;
  if (pb->dtype != FASTMAX_BF16 || pb->d != 64 || pb->order != 1 || pb->causal) return false;
  if (!a->o.ptr || a->state_in || a->state_out) return false;
  if (pb->nq <= 0 || pb->nk <= 0) return false;
  if ((long long)pb->batch * pb->heads < 64) return false;   // one CTA per head: fewer would leave most SMs idle
  return true;
}

static int tc_p1_forward(const fastmax_problem* pb, const fastmax_forward_args* a, cudaStream_t st) {
  CUtensorMap tmq, tmk, tmv, tmo;
  if (!make_map(&tmq, a->q, pb->batch, pb->heads, pb->nq, 64, tc::CH, true) ||
      !make_map(&tmk, a->k, pb->batch, pb->heads, pb->nk, 64, tc::CH, true) ||
      !make_map(&tmv, a->v, pb->batch, pb->heads, pb->nk, 8, tc::CH, false) ||
      !make_map(&tmo, a->o, pb->batch, pb->heads, pb->nq, 64, 32, true))   // output: 32-row boxes, one per epilogue warp
    return FASTMAX_TC_NOT_HANDLED;
  cudaError_t e = ensure_smem(tc::p1::p1_forward_kernel, tc::p1::SMEM_BYTES, 0);
  if (e != cudaSuccess) return report_cuda_error(e);
  tc::p1::P1Params P{View{a->g.ptr, a->g.stride_b, a->g.stride_h, a->g.stride_n},
                     pb->heads, pb->nq, pb->nk, pb->a0, pb->a1 * pb->inv_temperature};
  {
    LaunchScope ls(KK_P1_FWD, st);
    tc::p1::p1_forward_kernel<<<dim3(pb->batch * pb->heads), tc::p1::THREADS, tc::p1::SMEM_BYTES, st>>>(tmq, tmk, tmv, tmo, P);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

static int launch_seg_scan(float* seg, int nseg, const fastmax_problem* pb, const float* init, float* total_out, bool reverse,
                           cudaStream_t st) {
  const long long n = (long long)(pb->order == 2 ? 64 * 36 + 65 : 65) * 68;
  const long long total = (long long)pb->heads * n;
  {
    LaunchScope ls(KK_STATE_SCAN, st);
    tc::seg_state_scan_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(seg, nseg, pb->heads, n, init, total_out, reverse ? 1 : 0);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

// forward of a long batch-1 sequence cut into segments (see tc_segments)
static int tc_forward_segmented(const fastmax_problem* pb, const fastmax_forward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  const int nseg = tc_segments(pb);
  if (ws_bytes < tc_forward_workspace(pb, a)) return FASTMAX_ERR_WORKSPACE;
  const fastmax_problem vp = seg_problem(pb, nseg);
  float* seg = (float*)ws;
  void* inner = (char*)ws + seg_state_bytes(pb, nseg);
  const size_t inner_bytes = ws_bytes - seg_state_bytes(pb, nseg);
  int rc = FASTMAX_OK;
  if (a->key_moments_in != nullptr) {   // (1) moments of every segment's keys: from an earlier call with the same k, v ...
    cudaError_t e = cudaMemcpyAsync(seg, a->key_moments_in, seg_state_bytes(pb, nseg), cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return report_cuda_error(e);
  } else {                              // ... or summed here
    fastmax_forward_args t{};
    t.q = seg_view(a->k, vp.nk); t.k = seg_view(a->k, vp.nk); t.v = seg_view(a->v, vp.nk);
    t.state_out = seg;
    rc = tc_forward(&vp, &t, inner, inner_bytes, st);
    if (rc != FASTMAX_OK) return rc == FASTMAX_TC_NOT_HANDLED ? FASTMAX_ERR_UNSUPPORTED : rc;
  }
  if (a->key_moments_out != nullptr && a->key_moments_out != a->key_moments_in) {
    cudaError_t e = cudaMemcpyAsync(a->key_moments_out, seg, seg_state_bytes(pb, nseg), cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return report_cuda_error(e);
  }
  rc = launch_seg_scan(seg, nseg, pb, a->state_in, a->state_out, false, st);   // (2) exclusive prefix, total = state_out
  if (rc != FASTMAX_OK) return rc;
  if (!a->o.ptr) return FASTMAX_OK;   // a state-only call ends here
  fastmax_forward_args m{};   // (3) every segment from its prefix
  m.q = seg_view(a->q, vp.nq); m.k = seg_view(a->k, vp.nk); m.v = seg_view(a->v, vp.nk);
  m.o = seg_view(a->o, vp.nq); m.g = seg_view(a->g, vp.nq);
  m.state_in = seg;
  rc = tc_forward(&vp, &m, inner, inner_bytes, st);
  return rc == FASTMAX_TC_NOT_HANDLED ? FASTMAX_ERR_UNSUPPORTED : rc;
}

bool tc_takes_forward(const fastmax_problem* pb, const fastmax_forward_args* a) {
  return tc_p1_supported(pb, a) || tc_forward_segmentable(pb, a) || tc_forward_supported(pb, a) || tc_forward_paddable(pb, a);
}
static bool tc_forward_paddable(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (!tc_narrow_head(pb) || pb->nk <= 0) return false;
  const bool want_o = a->o.ptr != nullptr;
  if (want_o ? (pb->nq <= 0 || !pad_view_ok(a->q) || !pad_view_ok(a->o) || !a->g.ptr) : !a->state_out) return false;
  if (!pad_view_ok(a->k) || !pad_view_ok(a->v)) return false;
  fastmax_problem pp;
  fastmax_forward_args in;
  size_t used;
  padded_forward(pb, a, nullptr, pp, in, used);
  return tc_takes_forward(&pp, &in);
}
// forward of a narrow-head call on zero-padded copies
static int tc_forward_padded(const fastmax_problem* pb, const fastmax_forward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (ws_bytes < tc_forward_workspace(pb, a)) return FASTMAX_ERR_WORKSPACE;
  fastmax_problem pp;
  fastmax_forward_args in;
  size_t used;
  padded_forward(pb, a, (char*)ws, pp, in, used);
  const bool want_o = a->o.ptr != nullptr;
  cudaError_t e = launch_pad(a->k, pb, pb->nk, in.k.ptr, st);
  if (e == cudaSuccess) e = launch_pad(a->v, pb, pb->nk, in.v.ptr, st);
  if (e == cudaSuccess && want_o) e = launch_pad(a->q, pb, pb->nq, in.q.ptr, st);
  if (e == cudaSuccess && a->state_in) e = launch_state_width(a->state_in, const_cast<float*>(in.state_in), pb, true, st);
  if (e != cudaSuccess) return report_cuda_error(e);
  const int rc = tc_forward(&pp, &in, (char*)ws + used, ws_bytes - used, st);
  if (rc != FASTMAX_OK) return rc == FASTMAX_TC_NOT_HANDLED ? (int)FASTMAX_ERR_UNSUPPORTED : rc;
  if (want_o) e = launch_unpad(in.o.ptr, pb, pb->nq, a->o, st);
  if (e == cudaSuccess && a->state_out) e = launch_state_width(in.state_out, a->state_out, pb, false, st);
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

size_t tc_key_moments_bytes(const fastmax_problem* pb, const fastmax_forward_args* a) {
  if (tc_forward_paddable(pb, a)) {
    fastmax_problem pp;
    fastmax_forward_args in;
    size_t used;
    padded_forward(pb, a, nullptr, pp, in, used);
    return tc_key_moments_bytes(&pp, &in);
  }
  return tc_forward_segmentable(pb, a) ? seg_state_bytes(pb, tc_segments(pb)) : 0;
}

int tc_forward(const fastmax_problem* pb, const fastmax_forward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (tc_forward_paddable(pb, a)) return tc_forward_padded(pb, a, ws, ws_bytes, st);
  if (tc_p1_supported(pb, a)) return tc_p1_forward(pb, a, st);
  if (tc_forward_segmentable(pb, a)) return tc_forward_segmented(pb, a, ws, ws_bytes, st);
  if (!tc_forward_supported(pb, a)) return FASTMAX_TC_NOT_HANDLED;
  if (ws_bytes < tc_forward_workspace(pb, a)) return FASTMAX_ERR_WORKSPACE;
  const bool want_o = a->o.ptr && pb->nq > 0;
  CUtensorMap tmq, tmk, tmv;
  if (!make_map(&tmk, a->k, pb->batch, pb->heads, pb->nk, 64, tc::CH, true) ||
      !make_map(&tmv, a->v, pb->batch, pb->heads, pb->nk, 8, tc::CH, false))
    return FASTMAX_TC_NOT_HANDLED;  // layout the copy engine cannot describe: the CUDA-core engine takes it
  if (want_o) {
    if (!make_map(&tmq, a->q, pb->batch, pb->heads, pb->nq, 64, tc::CH, true)) return FASTMAX_TC_NOT_HANDLED;
  } else {
    tmq = tmk;   // a state-only call applies nothing: the tile is loaded and never read
  }
  const int bh = pb->batch * pb->heads;
  const ScanGeom G = scan_geom(pb);
  float* oacc = (float*)ws;
  const size_t oacc_bytes = want_o ? ((size_t)bh * pb->nq * 68 * sizeof(float) + 255) / 256 * 256 : 0;
  __nv_bfloat16* kt = (__nv_bfloat16*)((char*)ws + oacc_bytes);
  CUtensorMap tmkt;
  if (!make_map_t(&tmkt, kt, bh, pb->nk, tokens_padded(pb->nk))) return FASTMAX_TC_NOT_HANDLED;
  cudaError_t e = cudaSuccess;
  if (want_o) e = cudaMemsetAsync(oacc, 0, (size_t)bh * pb->nq * 68 * sizeof(float), st);
  if (e == cudaSuccess) e = launch_transpose(a->k, pb->batch, pb->heads, pb->nk, 0, kt, st);
  if (e != cudaSuccess) return report_cuda_error(e);
  tc::FwdParams P{};
  P.oacc = oacc;
  P.heads = pb->heads;
  P.nq = pb->nq;
  P.nk = pb->nk;
  P.off = G.k0;
  P.nchunks = G.nch;
  P.c0 = pb->a0;
  P.c1 = pb->a1 * pb->inv_temperature;
  P.c2 = pb->order == 2 ? pb->a2 * pb->inv_temperature * pb->inv_temperature : 0.f;
  e = ensure_smem(tc::s2::scan_apply_kernel<false>, tc::s2::SMEM_BYTES, 1);
  if (e == cudaSuccess)
    e = ensure_smem(tc::intra_fwd_kernel, tc::I_SMEM_BYTES, 2);
  if (e != cudaSuccess) return report_cuda_error(e);
  // the scan and the intra-chunk kernel both ADD into the O' accumulator: independent, side by side
  const bool intra = want_o && pb->causal;
  cudaStream_t ss[2];
  std::unique_lock<std::mutex> side_lock;
  SideStreams* side = intra ? fork_streams(pb, st, 2, ss, side_lock) : nullptr;
  if (!intra) ss[0] = ss[1] = st;
  JoinOnExit guard{side, st, 2};
  {
    LaunchScope ls(KK_TC_FWD, ss[0]);
    tc::s2::ApplyParams A{};
    A.out = oacc; A.heads = pb->heads; A.nz = pb->nq; A.ny = pb->nk; A.z_shift = G.k0; A.y_shift = 0; A.nchunks = G.nch;
    A.c0 = P.c0; A.c1 = P.c1; A.c2 = P.c2;
    A.state_out = a->state_out; A.state_in = a->state_in;
    A.sc = make_sched(G, false, a->state_in != nullptr, want_o, a->state_out != nullptr);
    A.nslices = G.nslices; A.tps = G.tps; A.tile_first = G.tile_first; A.state_rows = G.state_rows;
    tc::s2::scan_apply_kernel<false><<<dim3(G.nslices * bh), tc::s2::THREADS, tc::s2::SMEM_BYTES, ss[0]>>>(tmq, tmkt, tmv, A);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return report_cuda_error(e);
  if (intra) {
    LaunchScope ls(KK_TC_INTRA_FWD, ss[1]);
    const int nch_k = (pb->nk + tc::CH - 1) / tc::CH;
    tc::intra_fwd_kernel<<<dim3(nch_k, 1, bh), tc::I_THREADS, tc::I_SMEM_BYTES, ss[1]>>>(tmq, tmk, tmv, P);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) {
    guard.joined = true;
    e = join_streams(side, st, 2);
  }
  if (e != cudaSuccess) return report_cuda_error(e);
  return want_o ? launch_finalize_fwd(pb, a, oacc, st) : FASTMAX_OK;
}

static int device_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static bool tc_backward_supported(const fastmax_problem* pb, const fastmax_backward_args* a) {
  if (!tc_common_supported(pb) || pb->nq <= 0) return false;
  const bool want_grads = a->dq.ptr || a->dk.ptr || a->dv.ptr;
  if (want_grads && !(a->dq.ptr && a->dk.ptr && a->dv.ptr)) return false;
  if (!want_grads && !a->dstate_out) return false;
  if (!pb->causal && (a->state_in || a->dstate_in)) return false;
  if (a->state_in && pb->nk != pb->nq) return false;   // see the phase discipline note at Sched
  // the dO' prologue reads o and dO two bf16 at a time
  for (const fastmax_tensor* t : {&a->o, &a->d_out})
    if (((uintptr_t)t->ptr & 3) || (t->stride_b & 1) || (t->stride_h & 1) || (t->stride_n & 1)) return false;
  return true;
}

struct TcBwdLayout {
  size_t dop, qt, kt, dq, dk, dv, total;
};
static void tc_bwd_layout(const fastmax_problem* pb, bool want_grads, TcBwdLayout& L) {
  const size_t bh = (size_t)pb->batch * pb->heads;
  const ScanGeom G = scan_geom(pb, true);
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  size_t off = 0;
  L.dop = off; off += up(bh * pb->nq * 80 * sizeof(__nv_bfloat16));
  L.qt = off; off += transposed_bytes((int)bh, G.k0 + pb->nq);  // q transposed, column = position of the query
  L.kt = off; if (want_grads) off += transposed_bytes((int)bh, pb->nk);  // k transposed
  L.dq = off; if (want_grads) off += up(bh * pb->nq * tc::ACC_LD * sizeof(float));
  L.dk = off; if (want_grads) off += up(bh * pb->nk * tc::ACC_LD * sizeof(float));
  L.dv = off; if (want_grads) off += up(bh * pb->nk * tc::ACC_LD * sizeof(float));
  L.total = off;
}

static bool tc_backward_segmentable(const fastmax_problem* pb, const fastmax_backward_args* a) {
  if (tc_segments(pb) <= 0) return false;
  if (!(a->dq.ptr && a->dk.ptr && a->dv.ptr) && !(a->dstate_out && !a->dq.ptr)) return false;   // gradients, or a state-only call
  for (const fastmax_tensor* t : {&a->o, &a->d_out})
    if (((uintptr_t)t->ptr & 3) || (t->stride_b & 1) || (t->stride_h & 1) || (t->stride_n & 1)) return false;
  return true;
}

size_t tc_backward_workspace(const fastmax_problem* pb, const fastmax_backward_args* a) {
  if (tc_backward_paddable(pb, a)) {
    fastmax_problem pp;
    fastmax_backward_args in;
    size_t used;
    padded_backward(pb, a, nullptr, pp, in, used);
    return used + tc_backward_workspace(&pp, &in) + 256;
  }
  if (tc_backward_segmentable(pb, a)) {
    const int nseg = tc_segments(pb);
    const fastmax_problem vp = seg_problem(pb, nseg);
    float dummy = 0.f;
    fastmax_backward_args in = *a;
    in.state_in = nullptr; in.dstate_in = nullptr;
    in.dstate_out = a->dq.ptr ? nullptr : &dummy;   // a state-only call: the gradient-moment call over the segments is the inner call
    in.key_moments_in = nullptr; in.grad_moments_in = nullptr; in.grad_moments_out = nullptr;
    fastmax_forward_args f{};
    f.q = a->k; f.k = a->k; f.v = a->v;
    f.state_out = &dummy;   // sizes the state-only inner call
    const size_t inner_f = tc_forward_workspace(&vp, &f), inner_b = tc_backward_workspace(&vp, &in);
    return 2 * seg_state_bytes(pb, nseg) + (inner_f > inner_b ? inner_f : inner_b);
  }
  if (!tc_backward_supported(pb, a)) return 0;
  TcBwdLayout L;
  tc_bwd_layout(pb, a->dq.ptr != nullptr, L);
  return L.total;
}

// backward of a long batch-1 sequence cut into segments (see tc_segments)
static int tc_backward_segmented(const fastmax_problem* pb, const fastmax_backward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  const int nseg = tc_segments(pb);
  if (ws_bytes < tc_backward_workspace(pb, a)) return FASTMAX_ERR_WORKSPACE;
  const fastmax_problem vp = seg_problem(pb, nseg);
  const size_t sb = seg_state_bytes(pb, nseg);
  float* segS = (float*)ws;
  float* segD = (float*)((char*)ws + sb);
  void* inner = (char*)ws + 2 * sb;
  const size_t inner_bytes = ws_bytes - 2 * sb;
  auto fix = [](int rc) { return rc == FASTMAX_TC_NOT_HANDLED ? (int)FASTMAX_ERR_UNSUPPORTED : rc; };
  int rc = FASTMAX_OK;
  const bool want_grads = a->dq.ptr != nullptr;
  if (want_grads) {   // key moments of every segment, exclusive prefix (what dq needs): handed over by the forward call, or summed here
    if (a->key_moments_in != nullptr) {
      cudaError_t e = cudaMemcpyAsync(segS, a->key_moments_in, sb, cudaMemcpyDeviceToDevice, st);
      if (e != cudaSuccess) return report_cuda_error(e);
    } else {
      fastmax_forward_args t{};
      t.q = seg_view(a->k, vp.nk); t.k = seg_view(a->k, vp.nk); t.v = seg_view(a->v, vp.nk);
      t.state_out = segS;
      rc = tc_forward(&vp, &t, inner, inner_bytes, st);
      if (rc != FASTMAX_OK) return fix(rc);
    }
    rc = launch_seg_scan(segS, nseg, pb, a->state_in, nullptr, false, st);
    if (rc != FASTMAX_OK) return rc;
  }
  fastmax_backward_args m{};
  m.q = seg_view(a->q, vp.nq); m.k = seg_view(a->k, vp.nk); m.v = seg_view(a->v, vp.nk);
  m.o = seg_view(a->o, vp.nq); m.g = seg_view(a->g, vp.nq); m.d_out = seg_view(a->d_out, vp.nq);
  if (a->grad_moments_in != nullptr) {   // gradient moments of every segment, exclusive suffix (what dk, dv need)
    cudaError_t e = cudaMemcpyAsync(segD, a->grad_moments_in, sb, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return report_cuda_error(e);
  } else {
    fastmax_backward_args gmom = m;
    gmom.dstate_out = segD;
    rc = tc_backward(&vp, &gmom, inner, inner_bytes, st);
    if (rc != FASTMAX_OK) return fix(rc);
  }
  if (a->grad_moments_out != nullptr && a->grad_moments_out != a->grad_moments_in) {
    cudaError_t e = cudaMemcpyAsync(a->grad_moments_out, segD, sb, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return report_cuda_error(e);
  }
  rc = launch_seg_scan(segD, nseg, pb, a->dstate_in, a->dstate_out, true, st);
  if (rc == FASTMAX_OK && !want_grads) return FASTMAX_OK;   // a state-only call ends here
  if (rc != FASTMAX_OK) return rc;
  m.dq = seg_view(a->dq, vp.nq); m.dk = seg_view(a->dk, vp.nk); m.dv = seg_view(a->dv, vp.nk);
  m.state_in = segS; m.dstate_in = segD;
  return fix(tc_backward(&vp, &m, inner, inner_bytes, st));
}

bool tc_takes_backward(const fastmax_problem* pb, const fastmax_backward_args* a) {
  return tc_backward_segmentable(pb, a) || tc_backward_supported(pb, a) || tc_backward_paddable(pb, a);
}
static bool tc_backward_paddable(const fastmax_problem* pb, const fastmax_backward_args* a) {
  if (!tc_narrow_head(pb) || pb->nq <= 0 || pb->nk <= 0) return false;
  for (const fastmax_tensor* t : {&a->q, &a->k, &a->v, &a->o, &a->d_out})
    if (!pad_view_ok(*t)) return false;
  const bool want_grads = a->dq.ptr != nullptr;
  if (want_grads ? (!pad_view_ok(a->dq) || !pad_view_ok(a->dk) || !pad_view_ok(a->dv)) : !a->dstate_out) return false;
  if (!a->g.ptr) return false;
  fastmax_problem pp;
  fastmax_backward_args in;
  size_t used;
  padded_backward(pb, a, nullptr, pp, in, used);
  return tc_takes_backward(&pp, &in);
}
static int tc_backward_padded(const fastmax_problem* pb, const fastmax_backward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (ws_bytes < tc_backward_workspace(pb, a)) return FASTMAX_ERR_WORKSPACE;
  fastmax_problem pp;
  fastmax_backward_args in;
  size_t used;
  padded_backward(pb, a, (char*)ws, pp, in, used);
  cudaError_t e = launch_pad(a->q, pb, pb->nq, in.q.ptr, st);
  if (e == cudaSuccess) e = launch_pad(a->k, pb, pb->nk, in.k.ptr, st);
  if (e == cudaSuccess) e = launch_pad(a->v, pb, pb->nk, in.v.ptr, st);
  if (e == cudaSuccess) e = launch_pad(a->o, pb, pb->nq, in.o.ptr, st);
  if (e == cudaSuccess) e = launch_pad(a->d_out, pb, pb->nq, in.d_out.ptr, st);
  if (e == cudaSuccess && a->state_in) e = launch_state_width(a->state_in, const_cast<float*>(in.state_in), pb, true, st);
  if (e == cudaSuccess && a->dstate_in) e = launch_state_width(a->dstate_in, const_cast<float*>(in.dstate_in), pb, true, st);
  if (e != cudaSuccess) return report_cuda_error(e);
  const int rc = tc_backward(&pp, &in, (char*)ws + used, ws_bytes - used, st);
  if (rc != FASTMAX_OK) return rc == FASTMAX_TC_NOT_HANDLED ? (int)FASTMAX_ERR_UNSUPPORTED : rc;
  if (a->dq.ptr) {
    e = launch_unpad(in.dq.ptr, pb, pb->nq, a->dq, st);
    if (e == cudaSuccess) e = launch_unpad(in.dk.ptr, pb, pb->nk, a->dk, st);
    if (e == cudaSuccess) e = launch_unpad(in.dv.ptr, pb, pb->nk, a->dv, st);
  }
  if (e == cudaSuccess && a->dstate_out) e = launch_state_width(in.dstate_out, a->dstate_out, pb, false, st);
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

size_t tc_grad_moments_bytes(const fastmax_problem* pb, const fastmax_backward_args* a) {
  if (tc_backward_paddable(pb, a)) {
    fastmax_problem pp;
    fastmax_backward_args in;
    size_t used;
    padded_backward(pb, a, nullptr, pp, in, used);
    return tc_grad_moments_bytes(&pp, &in);
  }
  return tc_backward_segmentable(pb, a) ? seg_state_bytes(pb, tc_segments(pb)) : 0;
}

int tc_backward(const fastmax_problem* pb, const fastmax_backward_args* a, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (tc_backward_paddable(pb, a)) return tc_backward_padded(pb, a, ws, ws_bytes, st);
  if (tc_backward_segmentable(pb, a)) return tc_backward_segmented(pb, a, ws, ws_bytes, st);
  if (!tc_backward_supported(pb, a)) return FASTMAX_TC_NOT_HANDLED;
  const bool want_grads = a->dq.ptr != nullptr;
  TcBwdLayout L;
  tc_bwd_layout(pb, want_grads, L);
  if (ws_bytes < L.total) return FASTMAX_ERR_WORKSPACE;
  const int bh = pb->batch * pb->heads;
  const ScanGeom G = scan_geom(pb, true);
  char* base = (char*)ws;
  __nv_bfloat16* dop = (__nv_bfloat16*)(base + L.dop);
  float* dqa = (float*)(base + L.dq);
  float* dka = (float*)(base + L.dk);
  float* dva = (float*)(base + L.dv);
  __nv_bfloat16* qt = (__nv_bfloat16*)(base + L.qt);
  __nv_bfloat16* kt = (__nv_bfloat16*)(base + L.kt);
  const int nqpos = G.k0 + pb->nq;    // positions up to the last query
  CUtensorMap tmq, tmk, tmv, tmdo, tmqt, tmkt;
  fastmax_tensor dopt{dop, (int64_t)pb->heads * pb->nq * 80, (int64_t)pb->nq * 80, 80};
  if (!make_map(&tmq, a->q, pb->batch, pb->heads, pb->nq, 64, tc::CH, true) ||
      !make_map(&tmk, a->k, pb->batch, pb->heads, pb->nk, 64, tc::CH, true) ||
      !make_map(&tmv, a->v, pb->batch, pb->heads, pb->nk, 8, tc::CH, false) ||
      !make_map(&tmdo, dopt, pb->batch, pb->heads, pb->nq, 8, tc::CH, false, 80) ||
      !make_map_t(&tmqt, qt, bh, nqpos, tokens_padded(nqpos)) ||
      (want_grads && !make_map_t(&tmkt, kt, bh, pb->nk, tokens_padded(pb->nk))))
    return FASTMAX_TC_NOT_HANDLED;
  cudaError_t e = cudaSuccess;
  {
    const long long nrows = (long long)bh * pb->nq;
    const int threads = 256;
    bool vec = true;  // 128-bit path: bases and strides of dO and o are multiples of 8 elements
    for (const fastmax_tensor* t : {&a->o, &a->d_out})
      if (((uintptr_t)t->ptr & 15) || (t->stride_b & 7) || (t->stride_h & 7) || (t->stride_n & 7)) vec = false;
    const unsigned blocks = (unsigned)((nrows * (vec ? 8 : 32) + threads - 1) / threads);
    LaunchScope ls(KK_PROLOGUE, st);
    if (vec)
      tc::bwd_prologue_bf16_vec_kernel<<<blocks, threads, 0, st>>>(View{a->d_out.ptr, a->d_out.stride_b, a->d_out.stride_h, a->d_out.stride_n},
                                                                   View{a->o.ptr, a->o.stride_b, a->o.stride_h, a->o.stride_n},
                                                                   View{a->g.ptr, a->g.stride_b, a->g.stride_h, a->g.stride_n}, dop,
                                                                   pb->nq, pb->heads, nrows);
    else
    tc::bwd_prologue_bf16_kernel<<<blocks, threads, 0, st>>>(View{a->d_out.ptr, a->d_out.stride_b, a->d_out.stride_h, a->d_out.stride_n},
                                                             View{a->o.ptr, a->o.stride_b, a->o.stride_h, a->o.stride_n},
                                                             View{a->g.ptr, a->g.stride_b, a->g.stride_h, a->g.stride_n}, dop,
                                                             pb->nq, pb->heads, nrows);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return report_cuda_error(e);
  const float c0 = pb->a0, c1 = pb->a1 * pb->inv_temperature;
  const float c2 = pb->order == 2 ? pb->a2 * pb->inv_temperature * pb->inv_temperature : 0.f;
  e = ensure_smem(tc::s2::scan_apply_kernel<true>, tc::s2::SMEM_BYTES, 3);
  if (e != cudaSuccess) return report_cuda_error(e);
  auto dv_params = [&](bool want_apply) {
    tc::s2::ApplyParams A{};
    A.out = want_apply ? dva : nullptr; A.heads = pb->heads; A.nz = pb->nk; A.ny = pb->nk; A.z_shift = 0; A.y_shift = G.k0;
    A.nchunks = G.nch; A.c0 = c0; A.c1 = c1; A.c2 = c2;
    A.state_out = a->dstate_out; A.state_in = a->dstate_in;
    A.sc = make_sched(G, true, a->dstate_in != nullptr, want_apply, a->dstate_out != nullptr);
    A.nslices = G.nslices; A.tps = G.tps; A.tile_first = G.tile_first; A.state_rows = G.state_rows;
    return A;
  };
  if (!want_grads) {
    // only the gradient moments are wanted (what a sequence-parallel rank publishes): the dv scan, updates only
    e = launch_transpose(a->q, pb->batch, pb->heads, pb->nq, G.k0, qt, st);
    if (e != cudaSuccess) return report_cuda_error(e);
    {
      LaunchScope ls(KK_TC_BWD_DV, st);
      tc::s2::scan_apply_kernel<true><<<dim3(G.nslices * bh), tc::s2::THREADS, tc::s2::SMEM_BYTES, st>>>(tmk, tmqt, tmdo, dv_params(false));
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
  }
  // The chain-rule scans rebalance registers between their warp groups with setmaxnreg; that only terminates if
  // the CTA was launched with the register count the budget in tc_scan3.cuh assumes.  Otherwise the CUDA-core
  // engine takes the call.
  static const bool chain_ok = [] {
    cudaFuncAttributes f0{}, f1{};
    return cudaFuncGetAttributes(&f0, tc::s3::scan_chain_kernel<false>) == cudaSuccess &&
           cudaFuncGetAttributes(&f1, tc::s3::scan_chain_kernel<true>) == cudaSuccess &&
           f0.numRegs >= tc::s3::REG_LAUNCH && f1.numRegs >= tc::s3::REG_LAUNCH;
  }();
  if (!chain_ok) return FASTMAX_TC_NOT_HANDLED;
  e = ensure_smem(tc::s3::scan_chain_kernel<false>, tc::s3::SMEM_BYTES, 4);
  if (e == cudaSuccess)
    e = ensure_smem(tc::s3::scan_chain_kernel<true>, tc::s3::SMEM_BYTES, 5);
  if (e == cudaSuccess)
    e = ensure_smem(tc::intra_bwd_pipe_kernel, tc::IP_SMEM_BYTES, 6);
  if (e != cudaSuccess) return report_cuda_error(e);
  // Causal: the intra-chunk kernel goes first: it STORES its part into every row of the three accumulators (no
  // memset).  It fills all SMs by itself (one CTA per SM), so nothing is lost by letting the scans wait for it.  The
  // three scans then ADD on top with reduce operations, side by side: dv on the caller's stream, dq and dk on side
  // streams.  An accumulator is cast to its output as soon as its scan is done, on that scan's stream, so the casts
  // overlap the tails of the scans that are still running.  The transposed copies are only read by the scans: they
  // are made on the side streams while the intra-chunk kernel (which leaves the memory system idle) runs.
  // Non-causal: no chunk holds both queries and keys, so there is no intra-chunk term; the accumulators are zeroed.
  cudaStream_t ss[3];
  std::unique_lock<std::mutex> side_lock;
  SideStreams* side = fork_streams(pb, st, 3, ss, side_lock);
  JoinOnExit guard{side, st, 3};
  if (side) {
    e = launch_transpose(a->k, pb->batch, pb->heads, pb->nk, 0, kt, ss[1]);
    if (e == cudaSuccess) e = launch_transpose(a->q, pb->batch, pb->heads, pb->nq, G.k0, qt, ss[2]);
    if (e == cudaSuccess) e = cudaEventRecord(side->aux, ss[2]);   // the dv scan on the caller's stream reads q^T too
    if (e != cudaSuccess) return report_cuda_error(e);
  }
  if (pb->causal) {
    const int nch_k = (pb->nk + tc::CH - 1) / tc::CH;
    tc::IntraBwdParams I{dqa, dka, dva, pb->heads, pb->nq, pb->nk, G.k0, c0, c1, c2};
    LaunchScope ls(KK_TC_INTRA_BWD, ss[0]);
    const int nitems = nch_k * bh;
    const int ctas = nitems < device_sms() ? nitems : device_sms();   // persistent: one CTA per SM walks the items
    tc::intra_bwd_pipe_kernel<<<dim3(ctas), tc::IP_THREADS, tc::IP_SMEM_BYTES, ss[0]>>>(tmq, tmk, tmv, tmdo, I, nch_k, nitems);
    e = cudaGetLastError();
  } else {
    e = cudaMemsetAsync(dqa, 0, L.total - L.dq, ss[0]);   // the three accumulators are contiguous
  }
  if (e == cudaSuccess && side) {
    e = cudaEventRecord(side->mid, ss[0]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ss[1], side->mid, 0);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ss[2], side->mid, 0);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ss[0], side->aux, 0);
  } else if (e == cudaSuccess) {   // one stream: the copies simply follow
    e = launch_transpose(a->k, pb->batch, pb->heads, pb->nk, 0, kt, st);
    if (e == cudaSuccess) e = launch_transpose(a->q, pb->batch, pb->heads, pb->nq, G.k0, qt, st);
  }
  if (e != cudaSuccess) return report_cuda_error(e);
  auto chain_params = [&](bool dk) {
    tc::s3::ChainParams C{};
    C.out = dk ? dka : dqa;
    const fastmax_tensor& z = dk ? a->k : a->q;
    C.z = View{z.ptr, z.stride_b, z.stride_h, z.stride_n};
    C.heads = pb->heads; C.nz = dk ? pb->nk : pb->nq; C.nk = pb->nk; C.z_shift = dk ? 0 : G.k0; C.do_shift = G.k0;
    C.nchunks = G.nch; C.c1 = c1; C.c2 = c2;
    C.state_in = dk ? a->dstate_in : a->state_in;
    C.sc = make_sched(G, dk, C.state_in != nullptr, true, false);
    C.nslices = G.nslices; C.tps = G.tps; C.tile_first = G.tile_first; C.state_rows = G.state_rows;
    return C;
  };
  {
    LaunchScope ls(KK_TC_BWD_Q, ss[1]);
    tc::s3::scan_chain_kernel<false><<<dim3(G.nslices * bh), tc::s3::THREADS, tc::s3::SMEM_BYTES, ss[1]>>>(tmkt, tmv, tmdo, chain_params(false));
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return report_cuda_error(e);
  {
    // dk: the reverse chain-rule scan; dv: the reverse apply + update scan
    LaunchScope ls(KK_TC_BWD_KV, ss[2]);
    tc::s3::scan_chain_kernel<true><<<dim3(G.nslices * bh), tc::s3::THREADS, tc::s3::SMEM_BYTES, ss[2]>>>(tmqt, tmv, tmdo, chain_params(true));
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return report_cuda_error(e);
  {
    LaunchScope ls(KK_TC_BWD_DV, ss[0]);
    tc::s2::scan_apply_kernel<true><<<dim3(G.nslices * bh), tc::s2::THREADS, tc::s2::SMEM_BYTES, ss[0]>>>(tmk, tmqt, tmdo, dv_params(true));
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return report_cuda_error(e);
  int rc = launch_cast_out(pb, dqa, pb->nq, &a->dq, ss[1], tc::ACC_LD);
  if (rc == FASTMAX_OK) rc = launch_cast_out(pb, dka, pb->nk, &a->dk, ss[2], tc::ACC_LD);
  if (rc == FASTMAX_OK) rc = launch_cast_out(pb, dva, pb->nk, &a->dv, ss[0], tc::ACC_LD);
  if (rc != FASTMAX_OK) return rc;
  guard.joined = true;
  e = join_streams(side, st, 3);
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

int tc_wait_selftest(long long cycles, int code, cudaStream_t st) {
  tc::wait_selftest_kernel<<<1, 32, 0, st>>>(cycles, code);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FASTMAX_OK : report_cuda_error(e);
}

int tc_wait_histogram(int* out, int n) {
  int h[256];
  cudaError_t e = cudaMemcpyFromSymbol(h, g_tc_wait_hist, sizeof(h), 0, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return report_cuda_error(e);
  for (int i = 0; i < n && i < 256; ++i) out[i] = h[i];
  static const int zeros[256] = {0};
  cudaMemcpyToSymbol(g_tc_wait_hist, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice);
  return FASTMAX_OK;
}

int tc_device_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return report_cuda_error(e);
  *out = v;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice);
  }
  return FASTMAX_OK;
}

}  // namespace fm
