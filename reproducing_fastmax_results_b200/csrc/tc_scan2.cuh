// "Apply + update" scans with the Phi operands in tensor memory.  Included by tc_kernels.cu inside fm::tc.
//
// One kernel template serves two scans that have the same shape:
//   forward (DV = false), chunks ascending:    O'_c  = Phi(Q_c) Sb_{<c}           S  += Phi(K_c)^T [V_c | 1]
//   dv scan (DV = true),  chunks descending:   dV_c  = Phi(K_c) dSb_{>c}[:, :64]  dS += Phi(Q_c)^T dO'_c
// In both, "Z" is the raw [token][64] tile whose Phi multiplies the state copy (Q | K), "X" the tile whose Phi^T
// builds the state (K | Q, read from a transposed copy [64][tokens]) and "Y" the 80-column right-hand side of the
// update ([V|1] | dO').  The intra-chunk (masked) terms are added by separate kernels.  Which chunks apply, which
// update and where the bf16 state copy is refreshed comes from the call's schedule (Sched, tc_kernels.cu): causal
// calls do both in every chunk, a non-causal call updates over the key chunks and then applies over the query
// chunks, a state-only call only updates; the scan may start from a caller-provided state and write its final one.
//
// Why tensor memory: an SS tcgen05.mma with N = 80 reads 4 KB of A and 2.5 KB of B from shared memory per K = 16
// step (52 clocks of the 128 B/clock shared-memory pipe against 40 clocks of math), and a Phi tile that goes
// through shared memory costs another write and the read again.  Here the Phi tiles never touch shared memory:
// CUDA cores compute them in registers and store them with tcgen05.st into TMEM, where tcgen05.mma reads its A
// operand (45 clocks per K = 16 step measured); shared memory only carries the B operands and the raw tiles.
//
// Per 128-token chunk and 128-row feature tile t of the CTA's slice (4 tiles, the last slice 3):
//     apply   OUT (128 tok x N)    += Phi_t(Z_c) (128 tok x 128 feat, TMEM)     * Sb_t (128 feat x N, smem)
//     update  S_t (128 feat x 80)  += Phi_t(X_c)^T (128 feat x 128 tok, TMEM)   * Y_c (128 tok x 80, smem)
// A operands go through a ring of three 32-column TMEM buffers (128 lanes x 64 bf16 = a 64-deep K slab, four MMAs).
// An apply slab holds 64 features of Phi(Z) (thread = token, from the raw tile); an update slab holds 64 tokens of
// Phi(X)^T (thread = feature, from the transposed tile, rows of 144 bytes); both cost two 128-bit shared loads
// per eight products.  Slab order per (chunk, tile): A0 U0 A1 U1 (A0 A1 U0 U1 in the last tile, so the output drain
// overlaps the updates); U0 U1 in a chunk that only updates (e.g. the first chunk, which has no earlier state),
// A0 A1 in a chunk that only applies.  Three producer sets of four
// warps each own one ring slot (set s makes the slabs s, s+3, ... of the slab sequence); two issuer warps issue the
// apply and the update MMAs (independent accumulator chains) and wait on per-kind `full` barriers; every barrier
// has one producer and one consumer, so no waiter is ever more than one phase away from the barrier it polls.
// Polynomial weights: an off-diagonal pair unit stands for (a,b) and (b,a), factor 2, which the apply slab carries
// exactly (x_a is doubled); slices of pair tiles only then scale their output by c2 once, in float32, when it is
// drained.  The slice that holds the linear/constant tile puts the weights into the bf16 state copy instead.
// The output partial of the slice is staged in shared memory and added to the float32 accumulator in global
// memory with one bulk reduce (cp.reduce.async.bulk) per consumer warp and chunk (its 32 rows).
// TMEM columns: 0..319 four state accumulators, 320..399 output accumulator, 400..495 the ring.
// Warp roles (608 threads): 0-3, 4-7, 8-11 producer sets, 12-15 consumers (state -> bf16 copy, output drain),
// 16 apply issuer, 17 update issuer, 18 TMA loader.  Every wait is bounded (abort flag + error code).
#pragma once

namespace s2 {

constexpr int NSETS = 3;                               // producer sets = ring slots
constexpr int THREADS = 32 * (4 * NSETS + 4 + 3);      // 608
constexpr int W_CONS = 4 * NSETS, W_MMA = W_CONS + 4, W_MMA2 = W_MMA + 1, W_TMA = W_MMA + 2;
constexpr int NRING = NSETS;
constexpr int KT_ROW = 144;                            // row pitch of the transposed tile: 64 tokens + 8 (bank spread)
constexpr int KT_BOX = 64 * KT_ROW;                    // 9216: one 64-token box, [64 dims][72 tokens]
constexpr int KT_BUF = 2 * KT_BOX;                     // 18432
constexpr int VPBUF = 10 * BLK;                        // Y buffer: 9 column blocks + one zero block
constexpr int OFF_SB = 0;                              // 4 x SB_TILE
constexpr int OFF_VP = OFF_SB + 4 * SB_TILE;           // 73728, 2 buffers
constexpr int OFF_RAWQ = OFF_VP + 2 * VPBUF;           // 114688, 2 x REGION, 128-byte swizzle
constexpr int OFF_KT = OFF_RAWQ + 2 * REGION;          // 147456, 2 x KT_BUF (two 64-token boxes each, not swizzled)
constexpr int OFF_BAR = OFF_KT + 2 * KT_BUF;           // 184320
constexpr int OFF_TAB = OFF_BAR + 352;                 // slab tables of the producer sets: [3 sets][3 kinds][3 bases] words
constexpr int OFF_OST = OFF_BAR + 512;                 // output staging for the bulk reduce: 128 rows x <= 68 floats
constexpr int OST_BYTES = CH * 68 * 4;                 // 34816
constexpr int SMEM_BYTES = OFF_OST + OST_BYTES + 1024;
static_assert(OFF_RAWQ % 1024 == 0 && OFF_KT % 128 == 0 && OFF_OST % 128 == 0, "tile alignment");
constexpr uint32_t COL_O = 320u, COL_A = 400u;
// barriers
constexpr int B_FULL_Q = 0, B_FULL_K = 3, B_EMPTY = 6, B_Q_READY = 9, B_Q_FREE = 11, B_KT_READY = 13, B_KT_FREE = 15,
              B_VP_READY = 17, B_VP_FREE = 19, B_SB_READY = 21, B_S_DONE = 25, B_A_DONE = 29, B_O_DONE = 33, B_O_FREE = 34,
              B_COUNT = 35;
static_assert(B_COUNT * 8 <= 320 && OFF_TAB + 27 * 4 <= OFF_OST, "barrier block layout");

struct ApplyParams {
  float* out;          // forward: O' accumulator [BH][nz][68]; dv scan: dV accumulator [BH][nz][ACC_LD = 68]
  int heads;
  int nz;              // rows of Z and of the output (forward: nq; dv scan: nk)
  int ny;              // forward: number of keys (rows of the ones column that are 1)
  int z_shift;         // Z row of chunk position p is p - z_shift (forward: nk - nq; dv scan: 0)
  int y_shift;         // Y row of chunk position p is p - y_shift (forward: 0; dv scan: nk - nq)
  int nchunks;
  float c0, c1, c2;
  float* state_out;        // optional: the final state (forward: moments of all keys; dv scan: gradient moments), float32
                           // [BH][state_rows][68] (exchange layout)
  const float* state_in;   // optional: the state the scan starts from (same layout); sc.h = 1
  Sched sc;                // which chunks apply / update
  int nslices;             // thread blocks per head (order 2: 5 slices of 4 tiles, or 7 of 3; order 1: 1)
  int tps;                 // feature tiles per slice (at most 4: the TMEM accumulators)
  int tile_first;          // first feature tile of the problem (order 2: 0; order 1: the linear/constant tile)
  int state_rows;          // rows of the exchange layout (order 2: 64 * 36 + 65; order 1: 65)
};

// A bounded wait gave up: count the wait site (first failure of the CTA only), raise the CTA's abort flag, set the
// device status word.
__device__ __noinline__ void fail_record(int code, volatile int* abort_flag) {
  if (*abort_flag == 0) atomicAdd(&g_tc_wait_hist[code & 255], 1);
  *abort_flag = 1;
  atomicExch(&g_tc_status, code);
}
__device__ __noinline__ bool wait_slow(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
  return mbar_wait_abortable(bar, parity, WAIT_CYCLES, abort_flag);
}
// Waits for the phase of parity `parity`; the common case (already complete) is one try_wait.
__device__ __forceinline__ bool wait_fast(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_slow(bar, parity, abort_flag);
}

// Slab j of tile (chunk, t): is it an apply slab, and which half (64 features / 64 tokens) does it hold?
__device__ __forceinline__ void slab_kind(bool first_chunk, bool last_tile, int j, bool& is_q, int& half) {
  if (first_chunk) { is_q = false; half = j; }
  else if (last_tile) { is_q = (j < 2); half = j & 1; }
  else { is_q = !(j & 1); half = j >> 1; }
}

// Row `row` of a 128-byte-swizzled tile with 128-byte rows: 16-byte chunk cc.
__device__ __forceinline__ uint4 sw_chunk(const uint8_t* tile, int row, int cc) {
  return *reinterpret_cast<const uint4*>(tile + row * 128 + ((cc ^ (row & 7)) << 4));
}

// Apply slab: 64 features x[8a+mi] * x[8b+ri] of token row l of the raw [token][64] tile -> 32 packed registers
// (register 4 mi + j holds ri = 2j, 2j + 1).  `dbl`: x[8a+mi] is doubled (exact) for an off-diagonal unit.
__device__ __forceinline__ void apply_pair_slab(uint32_t (&r)[32], const uint8_t* raw, int l, int a, int b, bool dbl) {
  uint4 xa4 = sw_chunk(raw, l, a);
  const uint4 xb4 = sw_chunk(raw, l, b);
  if (dbl) {
    const uint32_t two = 0x40004000u;  // bf16x2 (2, 2)
    xa4.x = hmul2_u32(xa4.x, two); xa4.y = hmul2_u32(xa4.y, two); xa4.z = hmul2_u32(xa4.z, two); xa4.w = hmul2_u32(xa4.w, two);
  }
  const uint32_t xa[4] = {xa4.x, xa4.y, xa4.z, xa4.w};
#pragma unroll
  for (int mi = 0; mi < 8; ++mi) {
    const uint32_t pr = xa[mi >> 1];
    const uint32_t bc = (mi & 1) ? __byte_perm(pr, pr, 0x3232) : __byte_perm(pr, pr, 0x1010);
    r[4 * mi + 0] = hmul2_u32(bc, xb4.x);
    r[4 * mi + 1] = hmul2_u32(bc, xb4.y);
    r[4 * mi + 2] = hmul2_u32(bc, xb4.z);
    r[4 * mi + 3] = hmul2_u32(bc, xb4.w);
  }
}
// Update slab: products x[i][tok] * x[j][tok] for the 64 tokens of one box of the transposed tile ([64 dims] rows of
// KT_ROW bytes, not swizzled: the pitch spreads consecutive rows over the banks) -> 32 packed registers
// (register 4 cc + jj holds tokens 8cc + 2jj, +1).
__device__ __forceinline__ void update_pair_slab(uint32_t (&r)[32], const uint8_t* box, int i, int j) {
  const uint4* ri = reinterpret_cast<const uint4*>(box + i * KT_ROW);
  const uint4* rj = reinterpret_cast<const uint4*>(box + j * KT_ROW);
#pragma unroll
  for (int cc = 0; cc < 8; ++cc) {
    const uint4 xi = ri[cc];
    const uint4 xj = rj[cc];
    r[4 * cc + 0] = hmul2_u32(xi.x, xj.x);
    r[4 * cc + 1] = hmul2_u32(xi.y, xj.y);
    r[4 * cc + 2] = hmul2_u32(xi.z, xj.z);
    r[4 * cc + 3] = hmul2_u32(xi.w, xj.w);
  }
}
__device__ __forceinline__ void copy_row_slab(uint32_t (&r)[32], const uint8_t* tile, int row) {  // swizzled tile
#pragma unroll
  for (int cc = 0; cc < 8; ++cc) {
    const uint4 x = sw_chunk(tile, row, cc);
    r[4 * cc + 0] = x.x; r[4 * cc + 1] = x.y; r[4 * cc + 2] = x.z; r[4 * cc + 3] = x.w;
  }
}
__device__ __forceinline__ void copy_trow_slab(uint32_t (&r)[32], const uint8_t* box, int row) {  // transposed box
  const uint4* rr = reinterpret_cast<const uint4*>(box + row * KT_ROW);
#pragma unroll
  for (int cc = 0; cc < 8; ++cc) {
    const uint4 x = rr[cc];
    r[4 * cc + 0] = x.x; r[4 * cc + 1] = x.y; r[4 * cc + 2] = x.z; r[4 * cc + 3] = x.w;
  }
}
__device__ __forceinline__ void fill_slab(uint32_t (&r)[32], uint32_t v) {
#pragma unroll
  for (int c = 0; c < 32; ++c) r[c] = v;
}

// One slab of a tile for TMEM lane `row`: apply slabs take row = token, update slabs row = feature of the tile.
// pr: block pairs (a0, b0, a1, b1), 4 bits each, of the tile's two 64-feature units.  xt: transposed tile.
__device__ __forceinline__ void make_slab(uint32_t (&r)[32], bool is_q, int half, bool lin, bool dbl_off, int row,
                                          const uint8_t* raw, const uint8_t* xt, uint32_t pr) {
  if (is_q) {
    if (!lin) {
      const int a = (half ? (pr >> 8) : pr) & 15, b = (half ? (pr >> 12) : (pr >> 4)) & 15;
      apply_pair_slab(r, raw, row, a, b, dbl_off && a != b);
    } else if (half == 0) copy_row_slab(r, raw, row);         // features 0..63 = x
    else { fill_slab(r, 0u); r[0] = 0x00003F80u; }            // feature 64 = 1, the rest 0
  } else {
    const uint8_t* box = xt + half * KT_BOX;
    if (!lin) {
      const uint32_t q = (row >> 6) ? (pr >> 8) : pr;
      update_pair_slab(r, box, 8 * (int)(q & 15) + ((row >> 3) & 7), 8 * (int)((q >> 4) & 15) + (row & 7));
    } else if (row < 64) copy_trow_slab(r, box, row);
    else fill_slab(r, row == 64 ? 0x3F803F80u : 0u);
  }
}

template <bool DV>
__global__ void __launch_bounds__(THREADS, 1)
scan_apply_kernel(const __grid_constant__ CUtensorMap tmz, const __grid_constant__ CUtensorMap tmxt,
                  const __grid_constant__ CUtensorMap tmy, const ApplyParams P) {
  constexpr int OUT_LD = 68;                  // floats per output row (forward: O' | g | pad; dv scan: ACC_LD)
  constexpr int N_APPLY = DV ? 64 : 80;       // columns of the apply MMA
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sb = sm + OFF_SB;
  uint8_t* vp = sm + OFF_VP;
  uint8_t* rawq = sm + OFF_RAWQ;
  uint8_t* kt = sm + OFF_KT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BAR);
  float* ost = reinterpret_cast<float*>(sm + OFF_OST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_BAR + 320);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BAR + 328);

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  // The five slices of a head are neighbours in the grid, so they run at about the same time and share the head's
  // q / k / v tiles through L2.  gridDim.x = 5 * batch * heads.
  const int head = (int)blockIdx.x / P.nslices, slice = (int)blockIdx.x - P.nslices * head;
  const int b_idx = head / P.heads, h_idx = head - b_idx * P.heads;
  const int tile0 = P.tile_first + slice * P.tps;
  const int ntl = (NTILES - tile0) < P.tps ? (NTILES - tile0) : P.tps;
  const int nch = P.nchunks;
  const Sched sc = P.sc;
  const bool lin_slice = (tile0 + ntl == NTILES);   // this slice holds the linear/constant tile: weights go into Sb
  auto chunk_of = [&](int i) -> int { return DV ? (nch - 1 - i) : i; };  // i-th chunk of the scan
  uint32_t* slab_tabs = reinterpret_cast<uint32_t*>(sm + OFF_TAB);

  if (tid == 0) {
    // arrivals are one per WARP (an elected lane after __syncwarp), not one per thread
    for (int i = 0; i < NRING; ++i) { mbar_init(&bars[B_FULL_Q + i], 4); mbar_init(&bars[B_FULL_K + i], 4); mbar_init(&bars[B_EMPTY + i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_Q_READY + i], 1);  mbar_init(&bars[B_Q_FREE + i], 4 * NSETS);
      mbar_init(&bars[B_KT_READY + i], 1); mbar_init(&bars[B_KT_FREE + i], 4 * NSETS);
      mbar_init(&bars[B_VP_READY + i], 1); mbar_init(&bars[B_VP_FREE + i], 1);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(&bars[B_SB_READY + i], 4); mbar_init(&bars[B_S_DONE + i], 1); mbar_init(&bars[B_A_DONE + i], 1); }
    mbar_init(&bars[B_O_DONE], 1);
    mbar_init(&bars[B_O_FREE], 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (tid >= 32 && tid < 32 + 27) {
    // Slab tables, one entry per thread.  A chunk's slab sequence depends on its kind: 0 = apply + update (per tile
    // A0 U0 A1 U1, in the last tile A0 A1 U0 U1 so the output drain overlaps the updates), 1 = update only (U0 U1),
    // 2 = apply only (A0 A1).  Entry [set][kind][base]: the slabs of such a chunk that fall into ring slot `set` when
    // the chunk's first slab has sequence index `base` (mod 3); 4 bits per slab (tile | apply << 2 | half << 3), their
    // count in bits 28..31.
    const int e = tid - 32, set = e / 9, kind = (e / 3) % 3, base = e % 3;
    uint32_t tab = 0, n = 0;
    const int nsl = (kind == 0 ? 4 : 2) * ntl;
    for (int i = 0; i < nsl; ++i) {
      if ((base + i) % NSETS != set) continue;
      int t, half;
      bool is_q;
      if (kind == 0) { t = i >> 2; slab_kind(false, t == ntl - 1, i & 3, is_q, half); }
      else { t = i >> 1; is_q = (kind == 2); half = i & 1; }
      tab |= (uint32_t)(t | ((is_q ? 1 : 0) << 2) | (half << 3)) << (4 * n);
      ++n;
    }
    slab_tabs[e] = tab | (n << 28);
  }
  if (w == 0) tmem_alloc(tmem_slot, 512);
  // the MMAs read one column block past the nine stored ones of each B operand: keep those bytes finite
  for (int i = tid; i < (4 * SB_TILE + 2 * VPBUF) / 16; i += THREADS) reinterpret_cast<uint4*>(sb)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto WAIT = [&](int bar, uint32_t n) -> bool {  // waits for completion number n (0-based) of the barrier
    return wait_fast(&bars[bar], n & 1u, abort_flag);
  };
  auto FAIL = [&](int code) { fail_record(code, abort_flag); };  // out of line: keeps the hot loops compact

  if (w < W_CONS) {
    // ================= producers: Phi slabs into the TMEM ring =================
    // Set s fills ring slot s, i.e. every slab whose index in the CTA's slab sequence is s (mod 3).
    const int set = w >> 2;
    const int row = (w & 3) * 32 + lane;  // TMEM lane: token (apply slab) or feature of the tile (update slab)
    const uint32_t slot_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16) + COL_A + 32u * set;
    uint64_t pairs = 0;                   // 16 bits per tile: block pairs (a0, b0, a1, b1) of its two 64-feature units
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int a0 = 0, b0 = 0, a1 = 0, b1 = 0;
      if (tile0 + t < NTILES - 1) { pair_decode(2 * (tile0 + t), 8, a0, b0); pair_decode(2 * (tile0 + t) + 1, 8, a1, b1); }
      pairs |= (uint64_t)(a0 | (b0 << 4) | (a1 << 8) | (b1 << 12)) << (16 * t);
    }
    uint32_t base = 0; // (index of the current chunk's first slab) mod 3
    uint32_t k = 0;    // slabs this set has produced = phase count of its slot
    bool ok = true;
    for (int ci = 0; ci < nch && ok; ++ci) {
      const int buf = ci & 1;
      if (!WAIT(B_KT_READY + buf, (uint32_t)(ci >> 1)) || !WAIT(B_Q_READY + buf, (uint32_t)(ci >> 1))) { FAIL(200); break; }
      const bool has_a = sc.A(ci), has_u = sc.U(ci);
      if (has_a || has_u) {
        const int kind = (has_a && has_u) ? 0 : (has_u ? 1 : 2);
        const uint8_t* raw = rawq + buf * REGION;
        const uint8_t* xt = kt + buf * KT_BUF;
        const uint32_t tab = slab_tabs[(set * 3 + kind) * 3 + (int)base];
        const int cnt = (int)(tab >> 28);
#pragma unroll 1
        for (int e = 0; e < cnt; ++e, ++k) {
          const uint32_t d4 = (tab >> (4 * e)) & 15u;
          const int t = (int)(d4 & 3u), half = (int)(d4 >> 3);
          const bool is_q = (d4 & 4u) != 0;
          const bool lin = lin_slice && t == ntl - 1;
          const uint32_t pr = (uint32_t)(pairs >> (16 * t)) & 0xffffu;
          uint32_t r[32];
          make_slab(r, is_q, half, lin, !lin_slice, row, raw, xt, pr);
          if (k > 0 && !WAIT(B_EMPTY + set, k - 1)) { FAIL(201); ok = false; break; }
          __syncwarp();
          tc_fence_after_sync();
          tmem_st32(slot_addr, r);
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[(is_q ? B_FULL_Q : B_FULL_K) + set]);
        }
        base = (base + (uint32_t)((kind == 0 ? 4 : 2) * ntl)) % NSETS;
      }
      if (ok) {
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars[B_Q_FREE + buf]);
          mbar_arrive(&bars[B_KT_FREE + buf]);
        }
      }
    }
  } else if (w < W_MMA) {
    // ================= consumers: state conversion and output drain =================
    const int l = (w & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((w & 3) * 32) << 16);
    float* obase = P.out + (long long)head * P.nz * OUT_LD;
    const float out_scale = lin_slice ? 1.f : P.c2;   // pair-tile slices: the common weight c2, applied once, exactly
    constexpr int ST_LD = 68;
    bool ok = true;
    // S_t (float32, TMEM) -> Sb_t (bf16, shared memory), the B operand of the apply MMAs
    auto convert_tile = [&](int t) {
      uint8_t* dst = sb + t * SB_TILE + l * 16;
      if (lin_slice) {  // weights inside the copy: c2 / 2 c2 per unit, c1 and c0 in the linear/constant tile
        const float wgt = tile_weight(tile0 + t, l, P.c0, P.c1, P.c2);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t r[32];
          tmem_ld32(lane_addr + 80u * t + 32u * part, r);
          tmem_ld_wait();
#pragma unroll
          for (int jb = 0; jb < 4; ++jb) store_block8(dst + (4 * part + jb) * BLK, &r[8 * jb], wgt);
        }
        uint32_t r8[8];
        tmem_ld8(lane_addr + 80u * t + 64u, r8);
        tmem_ld_wait();
        store_block8(dst + 8 * BLK, r8, wgt);
      } else {          // plain rounding: the weights are in the apply slabs (factor 2) and in the drain (c2)
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t r[32];
          tmem_ld32(lane_addr + 80u * t + 32u * part, r);
          tmem_ld_wait();
#pragma unroll
          for (int jb = 0; jb < 4; ++jb) store_block8_plain(dst + (4 * part + jb) * BLK, &r[8 * jb]);
        }
        uint32_t r8[8];
        tmem_ld8(lane_addr + 80u * t + 64u, r8);
        tmem_ld_wait();
        store_block8_plain(dst + 8 * BLK, r8);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_SB_READY + t]);
    };
    if (sc.h) {
      // The scan starts from the caller's state: its rows go into the TMEM accumulators (80 columns: 64 values, the
      // denominator moment, zeros) and the first bf16 copy is made from them.  The arrival on SB_READY releases both
      // issuers, so it also orders these tensor-memory stores before the first update MMA.
      const float* sbase = P.state_in + (long long)head * P.state_rows * ST_LD;
      for (int t = 0; t < ntl; ++t) {
        const int srow = 128 * (tile0 + t - P.tile_first) + l;
        uint32_t ra[32], rb[32], rc[16];
        if (srow < P.state_rows) {
          const float4* src = reinterpret_cast<const float4*>(sbase + (long long)srow * ST_LD);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 x = src[j], y = src[8 + j];
            ra[4 * j] = __float_as_uint(x.x); ra[4 * j + 1] = __float_as_uint(x.y); ra[4 * j + 2] = __float_as_uint(x.z); ra[4 * j + 3] = __float_as_uint(x.w);
            rb[4 * j] = __float_as_uint(y.x); rb[4 * j + 1] = __float_as_uint(y.y); rb[4 * j + 2] = __float_as_uint(y.z); rb[4 * j + 3] = __float_as_uint(y.w);
          }
          rc[0] = __float_as_uint(src[16].x);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ra[j] = rb[j] = 0u;
          rc[0] = 0u;
        }
#pragma unroll
        for (int j = 1; j < 16; ++j) rc[j] = 0u;
        tmem_st32(lane_addr + 80u * t, ra);
        tmem_st32(lane_addr + 80u * t + 32u, rb);
        tmem_st16(lane_addr + 80u * t + 64u, rc);
        tmem_st_wait();
        convert_tile(t);
      }
    }
    for (int ci = 0; ci < nch && ok; ++ci) {
      const int c = chunk_of(ci);
      const bool has_a = sc.A(ci), has_c = sc.C(ci);
      for (int t = 0; t < ntl && ok; ++t) {
        if (t == ntl - 1 && has_a) {  // the output of this chunk is complete once the last apply has finished
          if (!WAIT(B_O_DONE, (uint32_t)sc.na_before(ci))) { FAIL(220); ok = false; break; }
          __syncwarp();
          tc_fence_after_sync();
          uint32_t ra[32], rb[32], rc[8];
          tmem_ld32(lane_addr + COL_O, ra);
          tmem_ld32(lane_addr + COL_O + 32u, rb);
          if (!DV) tmem_ld8(lane_addr + COL_O + 64u, rc);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[B_O_FREE]);
          // partial of this slice -> staging rows in shared memory -> bulk reduce-adds into the float32 accumulator
          // (the chunk's rows are contiguous there); the copy engine does the adds, fully coalesced.  Every warp
          // owns its 32 rows from TMEM to the reduce, so the four warps never wait for one another here.
          if (lane == 0) bulk_wait_read_all();   // this warp's previous reduce has read its staging rows
          __syncwarp();
          {
            float4* rowp = reinterpret_cast<float4*>(ost + l * OUT_LD);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              rowp[j] = make_float4(__uint_as_float(ra[4 * j]) * out_scale, __uint_as_float(ra[4 * j + 1]) * out_scale,
                                    __uint_as_float(ra[4 * j + 2]) * out_scale, __uint_as_float(ra[4 * j + 3]) * out_scale);
              rowp[8 + j] = make_float4(__uint_as_float(rb[4 * j]) * out_scale, __uint_as_float(rb[4 * j + 1]) * out_scale,
                                        __uint_as_float(rb[4 * j + 2]) * out_scale, __uint_as_float(rb[4 * j + 3]) * out_scale);
            }
            rowp[16] = DV ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(__uint_as_float(rc[0]) * out_scale, 0.f, 0.f, 0.f);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const long long q0 = (long long)c * CH - P.z_shift;  // output row of staging row 0
            const int wr0 = (w & 3) * 32;                        // this warp's staging rows
            int r0 = q0 < 0 ? (int)(-q0 < CH ? -q0 : CH) : 0;
            const long long lim = (long long)P.nz - q0;
            int r1 = lim < CH ? (lim < 0 ? 0 : (int)lim) : CH;
            r0 = r0 > wr0 ? r0 : wr0;
            r1 = r1 < wr0 + 32 ? r1 : wr0 + 32;
            if (r1 > r0) {
              bulk_reduce_add_f32(obase + (q0 + r0) * OUT_LD, ost + r0 * OUT_LD, (uint32_t)(r1 - r0) * (uint32_t)(OUT_LD * 4));
              bulk_commit_group();
            }
          }
        }
        if (has_c) {  // the bf16 copy of S_t feeds the next apply
          // S_t is final (this chunk's update) and Sb_t is no longer read (the applies up to and including this chunk's)
          const int na_thr = sc.na_before(ci) + (has_a ? 1 : 0);
          if (!WAIT(B_S_DONE + t, (uint32_t)(sc.nc_before(ci) - sc.h)) || (na_thr > 0 && !WAIT(B_A_DONE + t, (uint32_t)(na_thr - 1)))) { FAIL(221); ok = false; break; }
          __syncwarp();
          tc_fence_after_sync();
          convert_tile(t);
        }
      }
    }
    if (P.state_out != nullptr && ok) {
      // The caller wants the final state: S_t is complete once the last update has finished.  Tile rows are the
      // state's rows (two 64-feature pair units per tile, then the linear rows and the constant); the values are
      // un-weighted sums, which is the exchange format.  Features were rounded to bf16 before the products were
      // summed in float32.
      float* sbase = P.state_out + (long long)head * P.state_rows * ST_LD;
      const int nu = sc.nu_total();
      // S_DONE completions: one per copy, then one for the last update unless that update was followed by a copy
      const int last_sd = sc.ncv_total() + sc.s_final - 1;
      for (int t = 0; t < ntl; ++t) {
        if (nu > 0 && last_sd >= 0 && !WAIT(B_S_DONE + t, (uint32_t)last_sd)) { FAIL(224); break; }
        __syncwarp();
        tc_fence_after_sync();
        uint32_t ra[32], rb[32], rc[8];
        if (nu > 0 || sc.h) {
          tmem_ld32(lane_addr + 80u * t, ra);
          tmem_ld32(lane_addr + 80u * t + 32u, rb);
          tmem_ld8(lane_addr + 80u * t + 64u, rc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ra[j] = rb[j] = 0u;
          rc[0] = 0u;
        }
        const int srow = 128 * (tile0 + t - P.tile_first) + l;
        if (srow < P.state_rows) {
          float4* dst = reinterpret_cast<float4*>(sbase + (long long)srow * ST_LD);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dst[j] = make_float4(__uint_as_float(ra[4 * j]), __uint_as_float(ra[4 * j + 1]), __uint_as_float(ra[4 * j + 2]),
                                 __uint_as_float(ra[4 * j + 3]));
            dst[8 + j] = make_float4(__uint_as_float(rb[4 * j]), __uint_as_float(rb[4 * j + 1]), __uint_as_float(rb[4 * j + 2]),
                                     __uint_as_float(rb[4 * j + 3]));
          }
          dst[16] = make_float4(__uint_as_float(rc[0]), 0.f, 0.f, 0.f);
        }
      }
    }
    if (lane == 0) bulk_wait_all();  // this warp's last reduce has landed before the CTA retires
  } else if (w == W_MMA || w == W_MMA2) {
    // ================= MMA issuers =================
    // Warp W_MMA issues the apply MMAs (apply slabs -> output), warp W_MMA2 the update MMAs (update slabs -> S_t); the
    // two accumulator chains are independent.  Both walk the whole slab sequence to know each slab's ring slot, but
    // wait only for their own slabs, on per-kind `full` barriers whose phases count that kind's slabs in the slot.
    // The whole warp runs the loop with warp-uniform values; one elected lane issues the instructions (elect.sync
    // with a full mask always picks the same lane, which tcgen05.commit relies on).
    const bool mine_q = (w == W_MMA);
    constexpr uint32_t IDESC_A = make_idesc_bf16(128, N_APPLY, 0, 1);  // A from TMEM (K-major), B MN-major
    constexpr uint32_t IDESC_U = make_idesc_bf16(128, 80, 0, 1);
    const uint32_t idesc = mine_q ? IDESC_A : IDESC_U;
    const uint64_t dB_V = make_smem_desc(smem_u32(vp), 128, 2048, 0);
    const uint64_t dB_S = make_smem_desc(smem_u32(sb), 128, 2048, 0);
    uint64_t* full = &bars[mine_q ? B_FULL_Q : B_FULL_K];
    uint32_t s0 = 0;       // ring slot of the first slab of the current tile
    uint32_t phases = 0;   // bit s: parity of the next phase of this issuer's `full` barrier of slot s
    bool ok = true;
    // one slab: wait for it, four MMAs (K = 64), release the ring slot (+ the tile / chunk level commits)
    auto issue = [&](uint32_t slot, uint32_t d, uint64_t b0, uint32_t first, uint64_t* done1, uint64_t* done2) -> bool {
      if (!wait_fast(&full[slot], (phases >> slot) & 1u, abort_flag)) return false;
      __syncwarp();
      phases ^= (1u << slot);
      tc_fence_after_sync();
      const uint32_t a0 = tmem_base + COL_A + 32u * slot;
      if (elect_one()) {
        mma_ts(d, a0, b0, idesc, first);
        mma_ts(d, a0 + 8u, b0 + 16u, idesc, 1u);
        mma_ts(d, a0 + 16u, b0 + 32u, idesc, 1u);
        mma_ts(d, a0 + 24u, b0 + 48u, idesc, 1u);
        mma_commit(&bars[B_EMPTY + slot]);
        if (done1) mma_commit(done1);
        if (done2) mma_commit(done2);
      }
      __syncwarp();
      return true;
    };
    auto wrap = [](uint32_t x) -> uint32_t { return x >= NRING ? x - NRING : x; };  // x < 2 * NRING
    for (int ci = 0; ci < nch && ok; ++ci) {
      const uint64_t dB_Vc = dB_V + (uint64_t)(((ci & 1) * VPBUF) >> 4);
      const bool has_a = sc.A(ci), has_u = sc.U(ci);
      const int nc = sc.nc_before(ci);     // copies of the state made so far: this chunk works with copy number nc - 1
      // the Y tile is loaded for every chunk; a chunk without an update still hands its buffer back (below)
      if (!mine_q && !WAIT(B_VP_READY + (ci & 1), (uint32_t)(ci >> 1))) { FAIL(233); break; }
      if (mine_q && has_a) {               // the output accumulator is free once the previous apply has been drained
        const int na = sc.na_before(ci);
        if (na > 0 && !WAIT(B_O_FREE, (uint32_t)(na - 1))) { FAIL(231); break; }
      }
      // Positions of this issuer's two slabs of a tile in the chunk's slab sequence (see the slab tables), for a tile
      // that is not the last one (p0, p1) and for the last one (q0, q1); everything the tile loop needs is fixed here
      // so that the loop itself stays as short as the MMA issue rate wants it.
      const bool both = has_a && has_u, mine = mine_q ? has_a : has_u;
      const uint32_t p0 = (both && !mine_q) ? 1u : 0u, p1 = both ? (mine_q ? 2u : 3u) : 1u;
      const uint32_t q0 = (both && !mine_q) ? 2u : 0u, q1 = both ? (mine_q ? 1u : 3u) : 1u;
      const uint32_t adv = both ? 1u : 2u;   // four (or two) slabs per tile, modulo the three ring slots
      const uint32_t acc0 = mine_q ? 0u : ((sc.nu_before(ci) > 0 || sc.h) ? 1u : 0u);   // the first update starts the accumulator
      const bool sd = sc.SD(ci);
      if (!mine) {
        for (int t = 0; t < ntl && (has_a || has_u); ++t) s0 = wrap(s0 + adv);
      } else {
        for (int t = 0; t < ntl && ok; ++t) {
          const bool last = (t == ntl - 1);
          // Sb_t holds the copy this chunk's apply reads; the update may overwrite S_t once that copy exists
          if (nc > 0 && !WAIT(B_SB_READY + t, (uint32_t)(nc - 1))) { FAIL(230); ok = false; break; }
          if (mine_q) {
            const uint32_t d = tmem_base + COL_O;
            const uint64_t b = dB_S + (uint64_t)((t * SB_TILE) >> 4);
            ok = issue(s0, d, b, t > 0 ? 1u : 0u, nullptr, nullptr) &&
                 issue(wrap(s0 + (last ? q1 : p1)), d, b + 64u, 1u, &bars[B_A_DONE + t], last ? &bars[B_O_DONE] : nullptr);
            if (!ok) FAIL(232);
          } else {
            const uint32_t d = tmem_base + 80u * t;
            ok = issue(wrap(s0 + (last ? q0 : p0)), d, dB_Vc, acc0, nullptr, nullptr) &&
                 issue(wrap(s0 + (last ? q1 : p1)), d, dB_Vc + 64u, 1u, sd ? &bars[B_S_DONE + t] : nullptr,
                       last ? &bars[B_VP_FREE + (ci & 1)] : nullptr);
            if (!ok) FAIL(234);
          }
          s0 = wrap(s0 + adv);
        }
      }
      if (ok && !mine_q && !has_u) {       // nothing of this chunk reads the Y buffer
        if (elect_one()) mma_commit(&bars[B_VP_FREE + (ci & 1)]);
        __syncwarp();
      }
    }
    // every MMA of this issuer has completed once its last commit has arrived
    if (ok && nch > 0) {
      if (!mine_q) {
        if (!wait_fast(&bars[B_VP_FREE + ((nch - 1) & 1)], (uint32_t)((nch - 1) >> 1) & 1u, abort_flag)) FAIL(235);
      } else if (sc.na_total() > 0) {
        if (!wait_fast(&bars[B_A_DONE + ntl - 1], (uint32_t)(sc.na_total() - 1) & 1u, abort_flag)) FAIL(236);
      }
    }
    tc_fence_after_sync();
  } else {
    // ================= TMA loader =================
    bool ok = true;
    for (int ci = 0; ci < nch && ok; ++ci) {
      const int pos0 = chunk_of(ci) * CH, buf = ci & 1;
      const uint32_t k = (uint32_t)(ci >> 1);
      if (k > 0 && !WAIT(B_Q_FREE + buf, k - 1)) { FAIL(240); break; }
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[B_Q_READY + buf], REGION);
        tma_load_4d(rawq + buf * REGION, &tmz, &bars[B_Q_READY + buf], 0, pos0 - P.z_shift, h_idx, b_idx);
      }
      if (k > 0 && !WAIT(B_KT_FREE + buf, k - 1)) { FAIL(241); break; }
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars[B_KT_READY + buf], KT_BUF);
        tma_load_3d(kt + buf * KT_BUF, &tmxt, &bars[B_KT_READY + buf], pos0, 0, head);
        tma_load_3d(kt + buf * KT_BUF + KT_BOX, &tmxt, &bars[B_KT_READY + buf], pos0 + 64, 0, head);
      }
      if (k > 0 && !WAIT(B_VP_FREE + buf, k - 1)) { FAIL(242); break; }
      uint8_t* vbuf = vp + buf * VPBUF;
      if (!DV) {
        for (int r = lane; r < CH; r += 32)  // the ones column of [V | 1] (zero for rows past the last key)
          *reinterpret_cast<uint4*>(vbuf + 8 * BLK + r * 16) = make_uint4((pos0 + r < P.ny) ? 0x00003F80u : 0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
        __syncwarp();
      }
      if (lane == 0) {
        constexpr int NBLK = DV ? 9 : 8;
        mbar_arrive_expect_tx(&bars[B_VP_READY + buf], NBLK * BLK);
#pragma unroll
        for (int i = 0; i < NBLK; ++i) tma_load_4d(vbuf + i * BLK, &tmy, &bars[B_VP_READY + buf], 8 * i, pos0 - P.y_shift, h_idx, b_idx);
      }
      __syncwarp();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (w == 0) tmem_dealloc(tmem_base, 512);
}

// x (batch, head, token, 64) bf16, any strides -> xt [batch*head][64][ntp]: column p of xt holds token p - shift of x
// (zero where there is none; ntp is a multiple of 64).  One block per (64-column group, batch*head).  The tile goes
// through shared memory as 32-bit words (two dims each) with a row pitch of 33 words, so both the row-wise stores
// and the column-wise loads spread over the banks.
__global__ void __launch_bounds__(256) transpose_tokens_kernel(View x, __nv_bfloat16* __restrict__ xt, int n, int ntp, int heads,
                                                               int shift) {
  __shared__ uint32_t tile[64 * 33];
  const int head = blockIdx.y, t0 = blockIdx.x * 64;
  const int b = head / heads, h = head - b * heads;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (long long)b * x.sb + (long long)h * x.sh;
  for (int idx = threadIdx.x; idx < 512; idx += 256) {
    const int r = idx >> 3, cv = idx & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    const int tok = t0 + r - shift;
    if (tok >= 0 && tok < n) v = *reinterpret_cast<const uint4*>(src + (long long)tok * x.sn + cv * 8);
    uint32_t* dstw = &tile[r * 33 + cv * 4];
    dstw[0] = v.x; dstw[1] = v.y; dstw[2] = v.z; dstw[3] = v.w;
  }
  __syncthreads();
  // thread = (pair of dims dp, group of 8 tokens tg): eight words -> two output rows of eight tokens
  const int dp = threadIdx.x >> 3, tg = threadIdx.x & 7;
  uint32_t wv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wv[e] = tile[(tg * 8 + e) * 33 + dp];
  uint4 lo, hi;   // dims 2 dp and 2 dp + 1
  lo.x = __byte_perm(wv[0], wv[1], 0x5410); hi.x = __byte_perm(wv[0], wv[1], 0x7632);
  lo.y = __byte_perm(wv[2], wv[3], 0x5410); hi.y = __byte_perm(wv[2], wv[3], 0x7632);
  lo.z = __byte_perm(wv[4], wv[5], 0x5410); hi.z = __byte_perm(wv[4], wv[5], 0x7632);
  lo.w = __byte_perm(wv[6], wv[7], 0x5410); hi.w = __byte_perm(wv[6], wv[7], 0x7632);
  __nv_bfloat16* dst = xt + ((long long)head * 64 + 2 * dp) * ntp + t0 + tg * 8;
  *reinterpret_cast<uint4*>(dst) = lo;
  *reinterpret_cast<uint4*>(dst + ntp) = hi;
}

}  // namespace s2
