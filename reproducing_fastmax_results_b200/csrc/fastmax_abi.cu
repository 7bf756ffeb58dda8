// C ABI of the Fastmax engine (declared in include/fastmax_b200.h): argument validation, workspace
// carving, and the launch sequences of forward, backward and normalisation.
#include <atomic>
#include <mutex>
#include <vector>
#include <initializer_list>
#include <cstdio>
#include <cstring>

#include "../../include/fastmax_b200.h"
#include "aux_kernels.cuh"
#include "launchers.cuh"
#include "tc_launchers.cuh"

namespace fm {

static std::atomic<uint64_t> g_launches{0};
static thread_local int g_last_cuda_error = 0;

// ---- optional per-kernel timing -----------------------------------------------------------------
struct ProfRec {
  int kind;
  cudaEvent_t a, b;
};
static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
static std::vector<ProfRec> g_prof_recs;
static thread_local cudaEvent_t g_prof_open = nullptr;

bool profiling_on() { return g_prof_on.load(std::memory_order_relaxed) != 0; }

void launch_begin(int kind, cudaStream_t st) {
  (void)kind;
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  cudaEvent_t a = nullptr;
  if (cudaEventCreate(&a) != cudaSuccess) return;
  cudaEventRecord(a, st);
  g_prof_open = a;
}
void launch_end(int kind, cudaStream_t st) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (g_prof_open == nullptr) return;
  cudaEvent_t b = nullptr;
  if (cudaEventCreate(&b) == cudaSuccess) {
    cudaEventRecord(b, st);
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof_recs.push_back(ProfRec{kind, g_prof_open, b});
  } else {
    cudaEventDestroy(g_prof_open);
  }
  g_prof_open = nullptr;
}
static const char* kKindNames[KK_COUNT] = {
    "moments_kv", "moments_qg", "state_scan", "scan_fwd", "scan_bwd_q", "scan_bwd_kv", "finalize_fwd",
    "bwd_prologue", "cast_out", "normalize", "tc_scan_fwd", "tc_scan_bwd_q", "tc_scan_bwd_kv", "tc_moments", "p1_fwd", "tc_intra_fwd", "tc_intra_bwd", "tc_transpose", "tc_scan_bwd_dv", "decode_step", "key_prologue", "output_noise", "tc_pad"};

static int sm_count() {
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

int report_cuda_error(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return FASTMAX_ERR_CUDA;
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline View to_view(const fastmax_tensor& t) { return View{t.ptr, t.stride_b, t.stride_h, t.stride_n}; }

struct Plan {
  int bh, d, rows, ld, order;
  long long n_state;       // floats per head state
  int npair_slices, nslices;
  int C;
  // key axis (causal: shared by queries)
  int k_chunks, k_nseg, k_cps;
  // query axis
  int q_chunks, q_nseg, q_cps;
};

// Segments per head for a call whose (head, slice) thread blocks alone would leave SMs idle.  `per_sm` thread blocks
// of the scan kernels are resident per SM (registers and shared memory: two at head dims up to 32, else one), so the time goes with (waves of thread blocks) x (chunks per segment): the count that
// minimises that product is taken, e.g. 9 segments (288 blocks = 1.95 waves of 148) rather than 10 (320 blocks =
// 2.16 waves, i.e. three rounds) for 32 blocks per segment.
static int pick_nseg(int bh, int nslices, int nchunks, int min_chunks_per_seg, int per_sm) {
  const long long ctas = (long long)bh * nslices;
  const int sms = sm_count() * per_sm;
  if (ctas >= sms || nchunks <= 0) return 1;
  int cap = nchunks / min_chunks_per_seg;
  if (cap < 1) cap = 1;
  const int limit = (int)((4ll * sms + ctas - 1) / ctas);   // up to about four waves
  if (cap > limit) cap = limit;
  int best = 1;
  long long best_cost = (long long)nchunks;                 // one wave, every chunk in sequence
  for (int want = 2; want <= cap; ++want) {
    const int cps = (nchunks + want - 1) / want;
    const int nseg = (nchunks + cps - 1) / cps;
    const long long waves = (ctas * nseg + sms - 1) / sms;
    const long long cost = waves * cps;
    if (cost < best_cost) { best_cost = cost; best = nseg; }
  }
  return best;
}

static void split(int nchunks, int want, int& nseg, int& cps) {
  if (nchunks <= 0) {
    nseg = 1;
    cps = 1;
    return;
  }
  cps = (nchunks + want - 1) / want;
  nseg = (nchunks + cps - 1) / cps;
}

static int make_plan(const fastmax_problem* pb, Plan& pl, bool backward = false) {
  if (!pb) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->batch <= 0 || pb->heads <= 0 || pb->nq < 0 || pb->nk < 0) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->dtype != FASTMAX_F32 && pb->dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->d != 16 && pb->d != 32 && pb->d != 64) return FASTMAX_ERR_UNSUPPORTED;
  if (pb->order != 1 && pb->order != 2) return FASTMAX_ERR_UNSUPPORTED;
  if (pb->causal && pb->nk < pb->nq) return FASTMAX_ERR_UNSUPPORTED;
  if ((long long)pb->batch * pb->heads > 65535) return FASTMAX_ERR_UNSUPPORTED;
  pl.bh = pb->batch * pb->heads;
  pl.d = pb->d;
  pl.order = pb->order;
  pl.rows = state_rows(pb->d, pb->order);
  pl.ld = state_ld(pb->d);
  pl.n_state = (long long)pl.rows * pl.ld;
  int nb = pb->d / 8, npairs = nb * (nb + 1) / 2;
  pl.npair_slices = pb->order == 2 ? (npairs + 3) / 4 : 0;
  pl.nslices = pl.npair_slices + 1;
  pl.C = 64;
  pl.k_chunks = (pb->nk + pl.C - 1) / pl.C;
  pl.q_chunks = (pb->nq + pl.C - 1) / pl.C;
  // causal scans pay one extra moment pass when split into segments: only split when the GPU would idle
  (void)backward;
  const int per_sm = pb->d <= 32 ? 2 : 1;   // thread blocks of the scan kernels resident per SM, see scan_min_blocks
  int want_k = pick_nseg(pl.bh, pl.nslices, pl.k_chunks, pb->causal ? 8 : 2, per_sm);
  int want_q = pick_nseg(pl.bh, pl.nslices, pl.q_chunks, 2, per_sm);
  split(pl.k_chunks, want_k, pl.k_nseg, pl.k_cps);
  split(pl.q_chunks, want_q, pl.q_nseg, pl.q_cps);
  return FASTMAX_OK;
}

static int check_view(const fastmax_tensor& t, int dtype, bool need_vec) {
  if (!t.ptr) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (need_vec) {
    size_t es = dtype == FASTMAX_F32 ? 4 : 2;
    if (((uintptr_t)t.ptr) % 16) return FASTMAX_ERR_MISALIGNED;
    if ((t.stride_b * (long long)es) % 16 || (t.stride_h * (long long)es) % 16 || (t.stride_n * (long long)es) % 16)
      return FASTMAX_ERR_MISALIGNED;
  }
  return FASTMAX_OK;
}

#define FM_CUDA(expr)                         \
  do {                                        \
    cudaError_t e__ = (expr);                 \
    if (e__ != cudaSuccess) {                 \
      g_last_cuda_error = (int)e__;           \
      return FASTMAX_ERR_CUDA;                \
    }                                         \
  } while (0)

static cudaError_t launch_scan(int d, int dtype, int mode, bool causal, const ScanParams& P, dim3 grid, cudaStream_t st) {
  switch (d) {
    case 16: return launch_scan_d<16>(dtype, mode, causal, P, grid, st);
    case 32: return launch_scan_d<32>(dtype, mode, causal, P, grid, st);
    default: return launch_scan_d<64>(dtype, mode, causal, P, grid, st);
  }
}
static cudaError_t launch_moments(int d, int dtype, int src, const MomentParams& P, dim3 grid, cudaStream_t st) {
  switch (d) {
    case 16: return launch_moments_d<16>(dtype, src, P, grid, st);
    case 32: return launch_moments_d<32>(dtype, src, P, grid, st);
    default: return launch_moments_d<64>(dtype, src, P, grid, st);
  }
}

static void fill_coeffs(const fastmax_problem* pb, ScanParams& P) {
  P.c0 = pb->a0;
  P.c1 = pb->a1 * pb->inv_temperature;
  P.c2 = pb->order == 2 ? pb->a2 * pb->inv_temperature * pb->inv_temperature : 0.f;
  P.inv_temp = pb->inv_temperature;
}

// Builds the initial state of every segment of a scan over the key axis (causal) or the single total
// state (non-causal).  seg buffer: [bh][nseg][n_state].  Returns through P the seg_state pointers.
//   src MOM_KV: Phi(K)^T [V|1]          (forward direction: exclusive prefix)
//   src MOM_QG: Phi(Q)^T dO'            (reverse direction: exclusive suffix)
// raw_in: the per-segment sums of an earlier call with the same x and v (the moment pass is skipped); raw_out: receives them.
static int build_segment_states(const fastmax_problem* pb, const Plan& pl, int src, const View& x, const View& v,
                                const float* dop, float* segbuf, int nseg, int cps, int nchunks,
                                const float* init, float* total_out, int scan_op, cudaStream_t st,
                                const float* raw_in = nullptr, float* raw_out = nullptr) {
  const size_t raw_bytes = (size_t)pl.bh * nseg * pl.n_state * sizeof(float);
  if (raw_in != nullptr) {
    FM_CUDA(cudaMemcpyAsync(segbuf, raw_in, raw_bytes, cudaMemcpyDeviceToDevice, st));
    if (raw_out != nullptr && raw_out != raw_in) FM_CUDA(cudaMemcpyAsync(raw_out, raw_in, raw_bytes, cudaMemcpyDeviceToDevice, st));
    long long total = (long long)pl.bh * pl.n_state;
    {
      LaunchScope ls(KK_STATE_SCAN, st);
      state_scan_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(segbuf, nseg, pl.n_state, init, total_out, scan_op, total);
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  MomentParams M{};
  M.x = x;
  M.v = v;
  M.dop = dop;
  M.seg_total = segbuf;
  M.heads = pb->heads;
  if (src == MOM_KV) {
    M.nrows_x = pb->nk;
    M.nrows_y = pb->nk;
    M.x_shift = 0;
  } else {
    M.nrows_x = pb->nq;
    M.nrows_y = pb->nq;
    M.x_shift = pb->causal ? pb->nk - pb->nq : 0;
  }
  M.order = pb->order;
  M.nchunks = nchunks;
  M.chunks_per_seg = cps;
  M.nseg = nseg;
  M.npair_slices = pl.npair_slices;
  dim3 grid(pl.nslices, nseg, pl.bh);
  FM_CUDA(launch_moments(pb->d, pb->dtype, src, M, grid, st));
  if (raw_out != nullptr) FM_CUDA(cudaMemcpyAsync(raw_out, segbuf, raw_bytes, cudaMemcpyDeviceToDevice, st));
  long long total = (long long)pl.bh * pl.n_state;
  int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  {
    LaunchScope ls(KK_STATE_SCAN, st);
    state_scan_kernel<<<(unsigned)blocks, threads, 0, st>>>(segbuf, nseg, pl.n_state, init, total_out, scan_op, total);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

// a view whose rows can take 4-element vector stores
static bool vec4_ok(const fastmax_tensor& t, int dtype) {
  const size_t es = dtype == FASTMAX_F32 ? 4 : 2;
  const size_t al = 4 * es;
  return ((uintptr_t)t.ptr % al) == 0 && ((size_t)t.stride_b * es) % al == 0 && ((size_t)t.stride_h * es) % al == 0 &&
         ((size_t)t.stride_n * es) % al == 0;
}

// a bf16 view whose rows can take 8-element (128-bit) stores
static bool bf16x8_ok(const fastmax_tensor& t, int dtype, int d) {
  return dtype == FASTMAX_BF16 && (d & 7) == 0 && ((uintptr_t)t.ptr & 15) == 0 && (t.stride_b & 7) == 0 && (t.stride_h & 7) == 0 &&
         (t.stride_n & 7) == 0;
}

int launch_cast_out(const fastmax_problem* pb, const float* acc, int n, const fastmax_tensor* out, cudaStream_t st, int acc_ld) {
  if (acc_ld <= 0) acc_ld = pb->d;
  const long long total = (long long)pb->batch * pb->heads * n * pb->d;
  if (total == 0) return FASTMAX_OK;
  const int threads = 256;
  if (bf16x8_ok(*out, pb->dtype, pb->d) && (acc_ld & 3) == 0 && (long long)n * pb->d / 8 < (1ll << 30)) {
    dim3 grid((unsigned)(((long long)n * (pb->d / 8) + threads - 1) / threads), (unsigned)(pb->batch * pb->heads));
    {
      LaunchScope ls(KK_CAST, st);
      cast_out_bf16x8_kernel<<<grid, threads, 0, st>>>(acc, pb->d, n, pb->heads, to_view(*out), acc_ld);
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  if (vec4_ok(*out, pb->dtype) && (long long)n * pb->d / 4 < (1ll << 30)) {
    dim3 grid((unsigned)(((long long)n * (pb->d / 4) + threads - 1) / threads), (unsigned)(pb->batch * pb->heads));
    {
      LaunchScope ls(KK_CAST, st);
      if (pb->dtype == FASTMAX_F32)
        cast_out_vec_kernel<float><<<grid, threads, 0, st>>>(acc, pb->d, n, pb->heads, to_view(*out), acc_ld);
      else
        cast_out_vec_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(acc, pb->d, n, pb->heads, to_view(*out), acc_ld);
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  {
    LaunchScope ls(KK_CAST, st);
    if (pb->dtype == FASTMAX_F32)
      cast_out_kernel<float><<<blocks, threads, 0, st>>>(acc, pb->d, n, pb->heads, to_view(*out), total, acc_ld);
    else
      cast_out_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(acc, pb->d, n, pb->heads, to_view(*out), total, acc_ld);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

int launch_finalize_fwd(const fastmax_problem* pb, const fastmax_forward_args* a, const float* oacc, cudaStream_t st) {
  const int bh = pb->batch * pb->heads;
  const int ld = state_ld(pb->d);
  long long total = (long long)bh * pb->nq * pb->d;
  int threads = 256;
  if (bf16x8_ok(a->o, pb->dtype, pb->d) && (long long)pb->nq * pb->d / 8 < (1ll << 30)) {
    dim3 grid((unsigned)(((long long)pb->nq * (pb->d / 8) + threads - 1) / threads), (unsigned)bh);
    {
      LaunchScope ls(KK_FINALIZE, st);
      finalize_fwd_bf16x8_kernel<<<grid, threads, 0, st>>>(oacc, ld, pb->d, pb->nq, pb->heads, to_view(a->o), to_view(a->g));
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  if (vec4_ok(a->o, pb->dtype) && (long long)pb->nq * pb->d / 4 < (1ll << 30)) {
    dim3 grid((unsigned)(((long long)pb->nq * (pb->d / 4) + threads - 1) / threads), (unsigned)bh);
    {
      LaunchScope ls(KK_FINALIZE, st);
      if (pb->dtype == FASTMAX_F32)
        finalize_fwd_vec_kernel<float><<<grid, threads, 0, st>>>(oacc, ld, pb->d, pb->nq, pb->heads, to_view(a->o), to_view(a->g));
      else
        finalize_fwd_vec_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(oacc, ld, pb->d, pb->nq, pb->heads, to_view(a->o), to_view(a->g));
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  unsigned blocks = (unsigned)((total + threads - 1) / threads);
  {
    LaunchScope ls(KK_FINALIZE, st);
    if (pb->dtype == FASTMAX_F32)
      finalize_fwd_kernel<float><<<blocks, threads, 0, st>>>(oacc, ld, pb->d, pb->nq, pb->heads, to_view(a->o), to_view(a->g), total);
    else
      finalize_fwd_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(oacc, ld, pb->d, pb->nq, pb->heads, to_view(a->o), to_view(a->g), total);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace fm

using namespace fm;

extern "C" {

int32_t fastmax_state_rows(int32_t d, int32_t order) { return state_rows(d, order); }
int32_t fastmax_state_ld(int32_t d) { return state_ld(d); }
size_t fastmax_state_bytes(const fastmax_problem* pb) {
  if (!pb) return 0;
  return (size_t)pb->batch * pb->heads * state_rows(pb->d, pb->order) * state_ld(pb->d) * sizeof(float);
}

const char* fastmax_status_string(int32_t s) {
  switch (s) {
    case FASTMAX_OK: return "ok";
    case FASTMAX_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FASTMAX_ERR_UNSUPPORTED: return "unsupported shape (head dim must be 16/32/64, order 1/2, causal needs nk >= nq)";
    case FASTMAX_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case FASTMAX_ERR_CUDA: return "CUDA runtime error";
    case FASTMAX_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case FASTMAX_ERR_MISALIGNED: return "tensor base or stride not 16-byte aligned";
    case FASTMAX_ERR_SCRATCH_LIMIT: return "the problem needs more scratch than the library's built-in static array holds";
  }
  return "unknown status";
}
int32_t fastmax_last_cuda_error(void) { return g_last_cuda_error; }
const char* fastmax_last_cuda_error_string(void) { return cudaGetErrorString((cudaError_t)g_last_cuda_error); }
const char* fastmax_version(void) { return "fastmax_b200 0.1 (sm_100a)"; }
uint64_t fastmax_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int32_t fastmax_check_status(void) {
  int v = 0;
  int rc = tc_device_status(&v);
  if (rc) return rc;
  return v ? FASTMAX_ERR_DEVICE_TIMEOUT : FASTMAX_OK;
}

int32_t fastmax_debug_wait_histogram(int32_t* out, int32_t n) {
  if (!out || n <= 0) return FASTMAX_ERR_INVALID_ARGUMENT;
  return tc_wait_histogram(out, n);
}

int32_t fastmax_debug_wait_selftest(void* stream) {
  // about a millisecond of SM clocks; wait-site code 99 is used by no production kernel
  return tc_wait_selftest(2000000ll, 99, (cudaStream_t)stream);
}

int32_t fastmax_profile_enable(int32_t on) {
  g_prof_on.store(on ? 1 : 0);
  return FASTMAX_OK;
}
int32_t fastmax_profile_kinds(void) { return KK_COUNT; }
const char* fastmax_profile_kind_name(int32_t kind) { return (kind >= 0 && kind < KK_COUNT) ? kKindNames[kind] : ""; }
int32_t fastmax_profile_collect(double* ms, uint64_t* count, int32_t nkinds) {
  std::vector<ProfRec> recs;
  {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    recs.swap(g_prof_recs);
  }
  for (int i = 0; i < nkinds; ++i) {
    ms[i] = 0.0;
    count[i] = 0;
  }
  int rc = FASTMAX_OK;
  for (auto& r : recs) {
    float t = 0.f;
    cudaError_t e = cudaEventSynchronize(r.b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.a, r.b);
    if (e != cudaSuccess) {
      g_last_cuda_error = (int)e;
      rc = FASTMAX_ERR_CUDA;
    } else if (r.kind >= 0 && r.kind < nkinds) {
      ms[r.kind] += t;
      count[r.kind] += 1;
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  return rc;
}

// ---------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------
struct FwdLayout {
  size_t oacc, seg, total;
};
static int fwd_layout(const fastmax_problem* pb, const fastmax_forward_args* a, const Plan& pl, FwdLayout& L) {
  size_t off = 0;
  L.oacc = off;
  if (a->o.ptr) off += align_up((size_t)pl.bh * pb->nq * pl.ld * sizeof(float), 256);
  L.seg = off;
  bool need_seg = !pb->causal || pl.k_nseg > 1 || a->state_out != nullptr;
  if (need_seg) off += align_up((size_t)pl.bh * pl.k_nseg * pl.n_state * sizeof(float), 256);
  L.total = off;
  return need_seg;
}

size_t fastmax_forward_workspace(const fastmax_problem* pb, const fastmax_forward_args* args) {
  Plan pl;
  if (!args || make_plan(pb, pl) != FASTMAX_OK) return 0;
  FwdLayout L;
  fwd_layout(pb, args, pl, L);
  size_t tc = tc_forward_workspace(pb, args);
  return (L.total > tc ? L.total : tc) + 256;
}

int32_t fastmax_forward_engine(const fastmax_problem* pb, const fastmax_forward_args* args) {
  Plan pl;
  if (!args || make_plan(pb, pl) != FASTMAX_OK) return 0;
  return tc_takes_forward(pb, args) ? 1 : 0;
}

size_t fastmax_key_moments_bytes(const fastmax_problem* pb, const fastmax_forward_args* args) {
  Plan pl;
  if (!args || make_plan(pb, pl) != FASTMAX_OK || pb->nk == 0) return 0;
  if (const size_t t = tc_key_moments_bytes(pb, args)) return t;   // a long sequence cut into segments for the tensor-memory kernels
  if (tc_takes_forward(pb, args)) return 0;   // the tensor-memory kernels take this call whole: no segment sums
  FwdLayout L;
  if (!fwd_layout(pb, args, pl, L)) return 0;
  return (size_t)pl.bh * pl.k_nseg * pl.n_state * sizeof(float);
}

int32_t fastmax_forward(const fastmax_problem* pb, const fastmax_forward_args* a, void* ws, size_t ws_bytes,
                        void* stream) {
  Plan pl;
  if (!a) return FASTMAX_ERR_INVALID_ARGUMENT;
  int rc = make_plan(pb, pl);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // no queries: there is no output to write, but a requested state_out is still produced
  const bool want_o = a->o.ptr != nullptr && pb->nq > 0;
  if (pb->nq == 0 && !a->state_out) return FASTMAX_OK;  // no queries, no state requested: nothing to do
  if (!a->o.ptr && !a->state_out) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (!pb->causal && a->state_in) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->nk > 0) {
    if ((rc = check_view(a->k, pb->dtype, true))) return rc;
    if ((rc = check_view(a->v, pb->dtype, true))) return rc;
  }
  if (want_o) {
    if ((rc = check_view(a->q, pb->dtype, true))) return rc;
    if ((rc = check_view(a->o, pb->dtype, false))) return rc;
  }
  if (ws_bytes < fastmax_forward_workspace(pb, a) || (ws_bytes && (!ws || ((uintptr_t)ws % 256))))
    return FASTMAX_ERR_WORKSPACE;

  int tcrc = tc_forward(pb, a, ws, ws_bytes, st);
  if (tcrc != FASTMAX_TC_NOT_HANDLED) return tcrc;

  FwdLayout L;
  const bool need_seg = fwd_layout(pb, a, pl, L);
  char* base = (char*)ws;
  float* oacc = (float*)(base + L.oacc);
  float* seg = (float*)(base + L.seg);

  const View q = to_view(a->q), k = to_view(a->k), v = to_view(a->v);
  if (need_seg) {
    if (pb->nk == 0) {
      FM_CUDA(cudaMemsetAsync(seg, 0, (size_t)pl.bh * pl.k_nseg * pl.n_state * sizeof(float), st));
      if (a->state_out) {
        if (a->state_in)
          FM_CUDA(cudaMemcpyAsync(a->state_out, a->state_in, (size_t)pl.bh * pl.n_state * sizeof(float),
                                  cudaMemcpyDeviceToDevice, st));
        else
          FM_CUDA(cudaMemsetAsync(a->state_out, 0, (size_t)pl.bh * pl.n_state * sizeof(float), st));
      }
    } else {
      rc = build_segment_states(pb, pl, MOM_KV, k, v, nullptr, seg, pl.k_nseg, pl.k_cps, pl.k_chunks, a->state_in,
                                a->state_out, pb->causal ? SCAN_PREFIX : SCAN_TOTAL, st, a->key_moments_in, a->key_moments_out);
      if (rc) return rc;
    }
  }
  if (!want_o) return FASTMAX_OK;

  FM_CUDA(cudaMemsetAsync(oacc, 0, (size_t)pl.bh * pb->nq * pl.ld * sizeof(float), st));
  ScanParams P{};
  P.q = q; P.k = k; P.v = v;
  P.out0 = oacc;
  P.heads = pb->heads; P.nq = pb->nq; P.nk = pb->nk;
  P.off = pb->causal ? pb->nk - pb->nq : 0;
  P.order = pb->order; P.causal = pb->causal;
  P.npair_slices = pl.npair_slices;
  fill_coeffs(pb, P);
  if (pb->causal) {
    P.nchunks = pl.k_chunks; P.chunks_per_seg = pl.k_cps; P.nseg = pl.k_nseg;
    if (need_seg) {
      P.seg_state = seg; P.seg_state_head_stride = (long long)pl.k_nseg * pl.n_state; P.seg_state_seg_stride = pl.n_state;
    } else {
      P.seg_state = a->state_in; P.seg_state_head_stride = pl.n_state; P.seg_state_seg_stride = 0;
    }
  } else {
    P.nchunks = pl.q_chunks; P.chunks_per_seg = pl.q_cps; P.nseg = pl.q_nseg;
    P.seg_state = seg; P.seg_state_head_stride = (long long)pl.k_nseg * pl.n_state; P.seg_state_seg_stride = 0;
  }
  dim3 grid(pl.nslices, P.nseg, pl.bh);
  FM_CUDA(launch_scan(pb->d, pb->dtype, MODE_FWD, pb->causal != 0, P, grid, st));

  return launch_finalize_fwd(pb, a, oacc, st);
}

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
struct BwdLayout {
  size_t dop, dq, dk, dv, segS, segD, total;
  bool need_segS, need_segD, want_grads;
};
static void bwd_layout(const fastmax_problem* pb, const fastmax_backward_args* a, const Plan& pl, BwdLayout& L) {
  size_t off = 0;
  L.want_grads = a->dq.ptr || a->dk.ptr || a->dv.ptr;
  L.dop = off; off += align_up((size_t)pl.bh * pb->nq * pl.ld * sizeof(float), 256);
  L.dq = off; if (L.want_grads) off += align_up((size_t)pl.bh * pb->nq * pb->d * sizeof(float), 256);
  L.dk = off; if (L.want_grads) off += align_up((size_t)pl.bh * pb->nk * pb->d * sizeof(float), 256);
  L.dv = off; if (L.want_grads) off += align_up((size_t)pl.bh * pb->nk * pb->d * sizeof(float), 256);
  L.need_segS = L.want_grads && (!pb->causal || pl.k_nseg > 1);
  L.segS = off; if (L.need_segS) off += align_up((size_t)pl.bh * pl.k_nseg * pl.n_state * sizeof(float), 256);
  // gradient moments: causal -> segments over the key axis; non-causal -> over the query axis
  int nsegD = pb->causal ? pl.k_nseg : pl.q_nseg;
  L.need_segD = !pb->causal || pl.k_nseg > 1 || a->dstate_out != nullptr;
  L.segD = off; if (L.need_segD) off += align_up((size_t)pl.bh * nsegD * pl.n_state * sizeof(float), 256);
  L.total = off;
}

size_t fastmax_backward_workspace(const fastmax_problem* pb, const fastmax_backward_args* args) {
  Plan pl;
  if (!args || make_plan(pb, pl, true) != FASTMAX_OK) return 0;
  BwdLayout L;
  bwd_layout(pb, args, pl, L);
  size_t tc = tc_backward_workspace(pb, args);
  return (L.total > tc ? L.total : tc) + 256;
}

size_t fastmax_grad_moments_bytes(const fastmax_problem* pb, const fastmax_backward_args* args) {
  Plan pl;
  if (!args || make_plan(pb, pl, true) != FASTMAX_OK) return 0;
  if (const size_t t = tc_grad_moments_bytes(pb, args)) return t;
  if (tc_takes_backward(pb, args)) return 0;   // the tensor-memory kernels take this call whole: no segment sums
  BwdLayout L;
  bwd_layout(pb, args, pl, L);
  const int nsegD = pb->causal ? pl.k_nseg : pl.q_nseg;
  const int chunksD = pb->causal ? pl.k_chunks : pl.q_chunks;
  if (!L.need_segD || chunksD == 0) return 0;
  return (size_t)pl.bh * nsegD * pl.n_state * sizeof(float);
}

int32_t fastmax_backward(const fastmax_problem* pb, const fastmax_backward_args* a, void* ws, size_t ws_bytes,
                         void* stream) {
  Plan pl;
  if (!a) return FASTMAX_ERR_INVALID_ARGUMENT;
  int rc = make_plan(pb, pl, true);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  BwdLayout L;
  bwd_layout(pb, a, pl, L);
  if (!L.want_grads && !a->dstate_out) return FASTMAX_ERR_INVALID_ARGUMENT;
  // all three gradients or none (an empty tensor's pointer may be null: dq when nq == 0, dk and dv when nk == 0)
  if (L.want_grads && !((a->dq.ptr || pb->nq == 0) && ((a->dk.ptr && a->dv.ptr) || pb->nk == 0))) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (!pb->causal && (a->state_in || a->dstate_in)) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (pb->nq > 0) {
    if ((rc = check_view(a->q, pb->dtype, true))) return rc;
    if ((rc = check_view(a->o, pb->dtype, false))) return rc;
    if ((rc = check_view(a->g, FASTMAX_F32, false))) return rc;
    if ((rc = check_view(a->d_out, pb->dtype, false))) return rc;
  }
  if (L.want_grads) {
    if ((rc = check_view(a->k, pb->dtype, true))) return rc;
    if ((rc = check_view(a->v, pb->dtype, true))) return rc;
  }
  if (ws_bytes < fastmax_backward_workspace(pb, a) || !ws || ((uintptr_t)ws % 256)) return FASTMAX_ERR_WORKSPACE;
  if (pb->nq == 0 && pb->nk == 0) return FASTMAX_OK;
  if (pb->nq == 0) {
    // no query looks at these keys: dk = dv = 0, and the gradient moments pass through unchanged
    if (a->dstate_out) {
      const size_t nbytes = (size_t)pl.bh * pl.n_state * sizeof(float);
      if (a->dstate_in) FM_CUDA(cudaMemcpyAsync(a->dstate_out, a->dstate_in, nbytes, cudaMemcpyDeviceToDevice, st));
      else FM_CUDA(cudaMemsetAsync(a->dstate_out, 0, nbytes, st));
    }
    if (L.want_grads) {
      float* zk = (float*)((char*)ws + L.dk);
      float* zv = (float*)((char*)ws + L.dv);
      FM_CUDA(cudaMemsetAsync(zk, 0, L.segS - L.dk, st));
      if ((rc = launch_cast_out(pb, zk, pb->nk, &a->dk, st))) return rc;
      if ((rc = launch_cast_out(pb, zv, pb->nk, &a->dv, st))) return rc;
    }
    return FASTMAX_OK;
  }

  int tcrc = tc_backward(pb, a, ws, ws_bytes, st);
  if (tcrc != FASTMAX_TC_NOT_HANDLED) return tcrc;

  char* base = (char*)ws;
  float* dop = (float*)(base + L.dop);
  float* dqa = (float*)(base + L.dq);
  float* dka = (float*)(base + L.dk);
  float* dva = (float*)(base + L.dv);
  float* segS = (float*)(base + L.segS);
  float* segD = (float*)(base + L.segD);
  const View q = to_view(a->q), k = to_view(a->k), v = to_view(a->v);

  // dO' = [dO/g, -(dO.o)/g]
  if (pb->nq > 0) {
    long long nrows = (long long)pl.bh * pb->nq;
    int threads = 256;
    unsigned blocks = (unsigned)((nrows * 32 + threads - 1) / threads);
    {
      LaunchScope ls(KK_PROLOGUE, st);
      if (pb->dtype == FASTMAX_F32)
        bwd_prologue_kernel<float><<<blocks, threads, 0, st>>>(to_view(a->d_out), to_view(a->o), to_view(a->g), dop, pl.ld, pb->d, pb->nq, pb->heads, nrows);
      else
        bwd_prologue_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(to_view(a->d_out), to_view(a->o), to_view(a->g), dop, pl.ld, pb->d, pb->nq, pb->heads, nrows);
    }
    FM_CUDA(cudaGetLastError());
  }

  // gradient moments (reverse direction)
  const int nsegD = pb->causal ? pl.k_nseg : pl.q_nseg;
  const int cpsD = pb->causal ? pl.k_cps : pl.q_cps;
  const int chunksD = pb->causal ? pl.k_chunks : pl.q_chunks;
  if (L.need_segD) {
    if (chunksD == 0) {
      FM_CUDA(cudaMemsetAsync(segD, 0, (size_t)pl.bh * nsegD * pl.n_state * sizeof(float), st));
    } else {
      rc = build_segment_states(pb, pl, MOM_QG, q, v, dop, segD, nsegD, cpsD, chunksD, a->dstate_in, a->dstate_out,
                                pb->causal ? SCAN_SUFFIX : SCAN_TOTAL, st, a->grad_moments_in, a->grad_moments_out);
      if (rc) return rc;
    }
  }
  if (!L.want_grads) return FASTMAX_OK;

  // key moments (forward direction) for dq
  if (L.need_segS) {
    if (pb->nk == 0) {
      FM_CUDA(cudaMemsetAsync(segS, 0, (size_t)pl.bh * pl.k_nseg * pl.n_state * sizeof(float), st));
    } else {
      rc = build_segment_states(pb, pl, MOM_KV, k, v, nullptr, segS, pl.k_nseg, pl.k_cps, pl.k_chunks, a->state_in,
                                nullptr, pb->causal ? SCAN_PREFIX : SCAN_TOTAL, st, a->key_moments_in);
      if (rc) return rc;
    }
  }
  FM_CUDA(cudaMemsetAsync(dqa, 0, L.segS - L.dq, st));  // dq, dk, dv accumulators are contiguous

  ScanParams P{};
  P.q = q; P.k = k; P.v = v; P.dop = dop;
  P.heads = pb->heads; P.nq = pb->nq; P.nk = pb->nk;
  P.off = pb->causal ? pb->nk - pb->nq : 0;
  P.order = pb->order; P.causal = pb->causal;
  P.npair_slices = pl.npair_slices;
  fill_coeffs(pb, P);

  // dq: forward-direction scan with S
  if (pb->nq > 0) {
    ScanParams A = P;
    A.out0 = dqa;
    if (pb->causal) {
      A.nchunks = pl.k_chunks; A.chunks_per_seg = pl.k_cps; A.nseg = pl.k_nseg;
      if (L.need_segS) {
        A.seg_state = segS; A.seg_state_head_stride = (long long)pl.k_nseg * pl.n_state; A.seg_state_seg_stride = pl.n_state;
      } else {
        A.seg_state = a->state_in; A.seg_state_head_stride = pl.n_state; A.seg_state_seg_stride = 0;
      }
    } else {
      A.nchunks = pl.q_chunks; A.chunks_per_seg = pl.q_cps; A.nseg = pl.q_nseg;
      A.seg_state = segS; A.seg_state_head_stride = (long long)pl.k_nseg * pl.n_state; A.seg_state_seg_stride = 0;
    }
    dim3 grid(pl.nslices, A.nseg, pl.bh);
    FM_CUDA(launch_scan(pb->d, pb->dtype, MODE_BWD_Q, pb->causal != 0, A, grid, st));
  }
  // dk, dv: reverse-direction scan with dS
  if (pb->nk > 0) {
    ScanParams B = P;
    B.out0 = dka; B.out1 = dva;
    B.nchunks = pl.k_chunks; B.chunks_per_seg = pl.k_cps; B.nseg = pl.k_nseg;
    if (pb->causal) {
      if (L.need_segD) {
        B.seg_state = segD; B.seg_state_head_stride = (long long)nsegD * pl.n_state; B.seg_state_seg_stride = pl.n_state;
      } else {
        B.seg_state = a->dstate_in; B.seg_state_head_stride = pl.n_state; B.seg_state_seg_stride = 0;
      }
    } else {
      B.seg_state = segD; B.seg_state_head_stride = (long long)nsegD * pl.n_state; B.seg_state_seg_stride = 0;
    }
    dim3 grid(pl.nslices, B.nseg, pl.bh);
    FM_CUDA(launch_scan(pb->d, pb->dtype, MODE_BWD_KV, pb->causal != 0, B, grid, st));
  }

  // casts
  if ((rc = launch_cast_out(pb, dqa, pb->nq, &a->dq, st))) return rc;
  if ((rc = launch_cast_out(pb, dka, pb->nk, &a->dk, st))) return rc;
  if ((rc = launch_cast_out(pb, dva, pb->nk, &a->dv, st))) return rc;
  return FASTMAX_OK;
}

// ---------------------------------------------------------------------------------------------------
// optional key prologue / output epilogue
// ---------------------------------------------------------------------------------------------------
int32_t fastmax_key_prologue(int32_t batch, int32_t heads, int32_t nk, int32_t d, int32_t dtype, float inv_temperature,
                             const fastmax_tensor* k, const float* rpe, void* stream) {
  if (!k || batch < 0 || heads < 0 || nk < 0) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (d != 16 && d != 32 && d != 64) return FASTMAX_ERR_UNSUPPORTED;
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  if ((long long)batch * heads * nk == 0) return FASTMAX_OK;
  int rc = check_view(*k, dtype, true);
  if (rc) return rc;
  if (rpe && ((uintptr_t)rpe & 15)) return FASTMAX_ERR_MISALIGNED;
  if ((long long)batch * heads > 65535) return FASTMAX_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = 256;
  dim3 grid((unsigned)(((long long)nk * (d / 4) + threads - 1) / threads), (unsigned)(batch * heads));
  {
    LaunchScope ls(KK_KEY_PROLOGUE, st);
    if (dtype == FASTMAX_F32) key_prologue_kernel<float><<<grid, threads, 0, st>>>(to_view(*k), rpe, inv_temperature, d, nk, heads);
    else key_prologue_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(to_view(*k), rpe, inv_temperature, d, nk, heads);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

int32_t fastmax_output_noise(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype, float scale,
                             const fastmax_tensor* x, const fastmax_tensor* noise, const fastmax_tensor* out, void* stream) {
  if (!x || !noise || !out || batch < 0 || heads < 0 || n < 0) return FASTMAX_ERR_INVALID_ARGUMENT;
  if (d != 16 && d != 32 && d != 64) return FASTMAX_ERR_UNSUPPORTED;
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  if ((long long)batch * heads * n == 0) return FASTMAX_OK;
  for (const fastmax_tensor* t : {x, noise, out}) {
    int rc = check_view(*t, dtype, true);
    if (rc) return rc;
  }
  if ((long long)batch * heads > 65535) return FASTMAX_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = 256;
  dim3 grid((unsigned)(((long long)n * (d / 4) + threads - 1) / threads), (unsigned)(batch * heads));
  {
    LaunchScope ls(KK_OUTPUT_NOISE, st);
    if (dtype == FASTMAX_F32) output_noise_kernel<float><<<grid, threads, 0, st>>>(to_view(*x), to_view(*noise), to_view(*out), scale, d, n, heads);
    else output_noise_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(to_view(*x), to_view(*noise), to_view(*out), scale, d, n, heads);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

// ---------------------------------------------------------------------------------------------------
// normalisation
// ---------------------------------------------------------------------------------------------------
// 128-bit normalisation kernels: head dim 16 / 32 / 64 and every view aligned for 16-byte row pieces
static bool norm_vec_ok(int d, int dtype, std::initializer_list<const fastmax_tensor*> views) {
  if (d != 16 && d != 32 && d != 64) return false;
  const size_t es = dtype == FASTMAX_F32 ? 4 : 2;
  for (const fastmax_tensor* t : views)
    if (((uintptr_t)t->ptr & 15) || ((size_t)t->stride_b * es) % 16 || ((size_t)t->stride_h * es) % 16 || ((size_t)t->stride_n * es) % 16)
      return false;
  return true;
}
#define FM_NORM_VEC(KERNEL, ITERS, ...)                                                                 \
  do {                                                                                                  \
    const dim3 vblocks((unsigned)(((long long)n * (d / 8) + threads * (ITERS) - 1) / (threads * (ITERS))),  \
                       (unsigned)(batch * heads));                                                      \
    if (dtype == FASTMAX_F32) {                                                                         \
      if (d == 64) KERNEL<float, 8><<<vblocks, threads, 0, st>>>(__VA_ARGS__);                          \
      else if (d == 32) KERNEL<float, 4><<<vblocks, threads, 0, st>>>(__VA_ARGS__);                     \
      else KERNEL<float, 2><<<vblocks, threads, 0, st>>>(__VA_ARGS__);                                  \
    } else {                                                                                            \
      if (d == 64) KERNEL<__nv_bfloat16, 8><<<vblocks, threads, 0, st>>>(__VA_ARGS__);                  \
      else if (d == 32) KERNEL<__nv_bfloat16, 4><<<vblocks, threads, 0, st>>>(__VA_ARGS__);             \
      else KERNEL<__nv_bfloat16, 2><<<vblocks, threads, 0, st>>>(__VA_ARGS__);                          \
    }                                                                                                   \
  } while (0)

// One launch with a thread-block cluster per (batch, head).  Used when there are enough heads to fill the device
// with such clusters; a few long heads keep the two-launch form, whose blocks spread over all tokens.
static int norm_cluster_size(int batch, int heads, int n, int d) {
  const long long bh = (long long)batch * heads;
  const int rows_per_iter = 256 / (d / 8);
  int cl = 8;
  while (cl > 1 && n < cl * rows_per_iter * 2) cl /= 2;
  if (bh * cl < 2LL * sm_count()) return 0;
  return cl;
}
#define FM_NORM_FUSED(KERNEL, CL, ...)                                                                  \
  do {                                                                                                  \
    cudaLaunchConfig_t cfg = {};                                                                        \
    cfg.gridDim = dim3((unsigned)(CL), (unsigned)(batch * heads));                                      \
    cfg.blockDim = dim3(256);                                                                           \
    cfg.stream = st;                                                                                    \
    cudaLaunchAttribute attr[1];                                                                        \
    attr[0].id = cudaLaunchAttributeClusterDimension;                                                   \
    attr[0].val.clusterDim.x = (unsigned)(CL);                                                          \
    attr[0].val.clusterDim.y = 1;                                                                       \
    attr[0].val.clusterDim.z = 1;                                                                       \
    cfg.attrs = attr;                                                                                   \
    cfg.numAttrs = 1;                                                                                   \
    cudaError_t fe;                                                                                     \
    if (dtype == FASTMAX_F32) {                                                                         \
      if (d == 64) fe = cudaLaunchKernelEx(&cfg, KERNEL<float, 8>, __VA_ARGS__);                        \
      else if (d == 32) fe = cudaLaunchKernelEx(&cfg, KERNEL<float, 4>, __VA_ARGS__);                   \
      else fe = cudaLaunchKernelEx(&cfg, KERNEL<float, 2>, __VA_ARGS__);                                \
    } else {                                                                                            \
      if (d == 64) fe = cudaLaunchKernelEx(&cfg, KERNEL<__nv_bfloat16, 8>, __VA_ARGS__);                \
      else if (d == 32) fe = cudaLaunchKernelEx(&cfg, KERNEL<__nv_bfloat16, 4>, __VA_ARGS__);           \
      else fe = cudaLaunchKernelEx(&cfg, KERNEL<__nv_bfloat16, 2>, __VA_ARGS__);                        \
    }                                                                                                   \
    FM_CUDA(fe);                                                                                        \
  } while (0)

int32_t fastmax_normalize_forward(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype, float lim,
                                  const fastmax_tensor* x, const fastmax_tensor* y, uint64_t* stats, void* stream) {
  if (!x || !y || !x->ptr || !y->ptr || !stats || batch <= 0 || heads <= 0 || n < 0 || d <= 0 || !(lim > 0.f))
    return FASTMAX_ERR_INVALID_ARGUMENT;
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  long long nrows = (long long)batch * heads * n;
  FM_CUDA(cudaMemsetAsync(stats, 0, (size_t)batch * heads * sizeof(uint64_t), st));
  if (nrows == 0) return FASTMAX_OK;
  int threads = 256;
  unsigned blocks = (unsigned)((nrows * 32 + threads - 1) / threads);
  unsigned long long* sp = reinterpret_cast<unsigned long long*>(stats);
  if (norm_vec_ok(d, dtype, {x, y}) && (long long)batch * heads <= 65535) {
    if (const int cl = norm_cluster_size(batch, heads, n, d)) {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_FUSED(norm_fused_vec_kernel, cl, to_view(*x), to_view(*y), (int)n, (int)heads, sp, lim);
      return FASTMAX_OK;
    }
    {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_VEC(norm_stats_vec_kernel, NORM_ITERS, to_view(*x), n, heads, sp, nrows);
    }
    {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_VEC(norm_apply_vec_kernel, 1, to_view(*x), to_view(*y), n, heads, sp, lim, nrows);
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  {
    LaunchScope ls(KK_NORMALIZE, st);
    if (dtype == FASTMAX_F32)
      norm_stats_kernel<float><<<blocks, threads, 0, st>>>(to_view(*x), d, n, heads, sp, nrows);
    else
      norm_stats_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(to_view(*x), d, n, heads, sp, nrows);
  }
  {
    LaunchScope ls(KK_NORMALIZE, st);
    if (dtype == FASTMAX_F32)
      norm_apply_kernel<float><<<blocks, threads, 0, st>>>(to_view(*x), to_view(*y), d, n, heads, sp, lim, nrows);
    else
      norm_apply_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(to_view(*x), to_view(*y), d, n, heads, sp, lim, nrows);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

int32_t fastmax_normalize_backward(int32_t batch, int32_t heads, int32_t n, int32_t d, int32_t dtype, float lim,
                                   const fastmax_tensor* y, const fastmax_tensor* dy, const fastmax_tensor* dx,
                                   const uint64_t* stats, float* scratch, void* stream) {
  if (!y || !dy || !dx || !y->ptr || !dy->ptr || !dx->ptr || !stats || !scratch || batch <= 0 || heads <= 0 ||
      n < 0 || d <= 0 || !(lim > 0.f))
    return FASTMAX_ERR_INVALID_ARGUMENT;
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16) return FASTMAX_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  long long nrows = (long long)batch * heads * n;
  FM_CUDA(cudaMemsetAsync(scratch, 0, (size_t)batch * heads * sizeof(float), st));
  if (nrows == 0) return FASTMAX_OK;
  int threads = 256;
  unsigned blocks = (unsigned)((nrows * 32 + threads - 1) / threads);
  const unsigned long long* sp = reinterpret_cast<const unsigned long long*>(stats);
  if (norm_vec_ok(d, dtype, {y, dy, dx}) && (long long)batch * heads <= 65535) {
    if (const int cl = norm_cluster_size(batch, heads, n, d)) {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_FUSED(norm_bwd_fused_vec_kernel, cl, to_view(*y), to_view(*dy), to_view(*dx), (int)n, (int)heads, sp, lim);
      return FASTMAX_OK;
    }
    {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_VEC(norm_bwd_dot_vec_kernel, NORM_ITERS, to_view(*y), to_view(*dy), n, heads, scratch, nrows);
    }
    {
      LaunchScope ls(KK_NORMALIZE, st);
      FM_NORM_VEC(norm_bwd_apply_vec_kernel, 1, to_view(*y), to_view(*dy), to_view(*dx), n, heads, sp, scratch, lim, nrows);
    }
    FM_CUDA(cudaGetLastError());
    return FASTMAX_OK;
  }
  {
    LaunchScope ls(KK_NORMALIZE, st);
    if (dtype == FASTMAX_F32)
      norm_bwd_dot_kernel<float><<<blocks, threads, 0, st>>>(to_view(*y), to_view(*dy), d, n, heads, scratch, nrows);
    else
      norm_bwd_dot_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(to_view(*y), to_view(*dy), d, n, heads, scratch, nrows);
  }
  {
    LaunchScope ls(KK_NORMALIZE, st);
    if (dtype == FASTMAX_F32)
      norm_bwd_apply_kernel<float><<<blocks, threads, 0, st>>>(to_view(*y), to_view(*dy), to_view(*dx), d, n, heads, sp, scratch, lim, nrows);
    else
      norm_bwd_apply_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(to_view(*y), to_view(*dy), to_view(*dx), d, n, heads, sp, scratch, lim, nrows);
  }
  FM_CUDA(cudaGetLastError());
  return FASTMAX_OK;
}

}  // extern "C"
