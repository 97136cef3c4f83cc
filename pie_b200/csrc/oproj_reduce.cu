// Output projection of a head-sharded layer with the sum over the ranks in its epilogue (sm_100a
// tcgen05 / TMEM, plain peer loads and stores over NVLink; no TMA or multicast on another GPU's memory).
//
//   out[n, hidden] = residual[n, hidden] + sum over ranks r of a_r[n, K_r] . w_r[hidden, K_r]^T
//
// is the reference's row-parallel o_proj, its all-reduce and the first residual connection
// (pie/src/pie_worker/model/llama3.py:693-709: linear on the local shard, dist.all_reduce, residual +
// attn_proj).  Every rank launches this kernel on its own shard in the same step; no collective follows.
//
// A tile is 128 tokens x NT hidden columns; tile t belongs to rank t mod world (its owner).  Every rank
// computes its partial sum of every tile (one pass over its w shard), accumulator in tensor memory, fp32.
//   * a tile owned by another rank: the epilogue stores the fp32 partial into the owner's staging area
//     (peer stores) and raises the owner's arrival flag for (tile, this rank);
//   * an owned tile: the epilogue waits (bounded) for the other ranks' partials, adds them in rank order to
//     its own (which never leaves tensor memory), adds the residual, rounds ONCE, stores the rows into the
//     output buffer of EVERY rank and raises every rank's completion flag of the tile.
// Before a CTA retires it waits for the completion flags of the tiles it computed, so the kernel's end
// means that this rank's output is whole.  The sum is the same bits on every rank (one rank computes it)
// and does not depend on timing (fixed order).
//
// The staging layout is private: within a tile, 16-byte pieces (4 fp32 columns) of the 128 rows are
// contiguous, so that the 32 rows of a warp store and load 512 contiguous bytes per instruction.  Warp w
// of the owner reads exactly the rows and columns that warp w of the sender wrote, so the flags are per
// warp and the epilogue warps never meet at a block-wide barrier.  On request the partials travel rounded to
// the 16-bit storage type (8 columns per piece): an all-reduce's bytes and numerics.  The owner's result rows
// go through a swizzled shared-memory tile of the warp and leave as 128-byte row pieces: a thread-per-row
// store would put 16-byte fragments, a row apart, on the link.
//
// All ranks must launch with the same sizes (and so the same grid): a CTA takes its tiles in increasing
// order on every rank, which is what keeps the waits free of cycles.  Flags carry the step number, which
// the caller increases from call to call; the output buffers of consecutive steps must alternate (a rank
// may run one step ahead of a rank that still reads the previous result).
// Roles as in the QKV kernel: warps 0-7 epilogue (thread = token row = TMEM lane; warps w and w + 4 share
// the rows and take half of the columns each), warp 8 TMA producer, warp 9 MMA issuer and TMEM owner.
// Every wait is bounded (2 s); on expiry the error word is set and all roles leave.
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace piekv {

namespace {

constexpr int kOBM = 128, kOBK = 64;
constexpr int kOTileBytes = kOBM * kOBK * 2;  // the a tile of a k-block: 128 rows x 64 16-bit elements
constexpr int kOEpiWarps = 8, kOProducerWarp = 8, kOMmaWarp = 9;
constexpr int kOThreads = 32 * (kOEpiWarps + 2);
constexpr int kOFlagsPerTile = kOEpiWarps;

struct OprojParams {
  int n, k, hidden;
  int world, rank, step;
  int slots;  // tiles an owner may hold: ceil(tiles / world)
  int stage16;  // partial sums travel rounded to the 16-bit storage type instead of fp32
  uint8_t *stage[PIEKV_MAX_PEERS];   // stage[r]: [world][slots][NT / 4][128][4] fp32 (or [NT / 8][128][8] 16-bit) on rank r
  int32_t *arrive[PIEKV_MAX_PEERS];  // arrive[r]: [slots][world][8] on rank r
  int32_t *done[PIEKV_MAX_PEERS];    // done[r]: [tiles][8] on rank r
  void *out[PIEKV_MAX_PEERS];        // out[r]: [n, hidden] on rank r
  const void *residual;              // nullable: [n, hidden] (this rank's copy; every rank holds the same)
  int64_t residual_stride;
  int32_t *err;
#ifdef PIEKV_OTRACE
  long long *trace;  // [CTAs][8]: clocks of epilogue warp 0 spent per phase
#endif
};

#ifdef PIEKV_OTRACE
#define OTRACE_DECL long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long tr_t = clock64();
#define OTRACE(i)                   \
  {                                 \
    const long long now = clock64(); \
    tr[i] += now - tr_t;            \
    tr_t = now;                     \
  }
#else
#define OTRACE_DECL
#define OTRACE(i)
#endif

__device__ __forceinline__ void st_release_sys(int32_t *p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t *p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T, int NT, int STAGES>
__global__ void __launch_bounds__(kOThreads, 1)
    oproj_reduce_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                        const __grid_constant__ OprojParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int kWTileBytes = NT * kOBK * 2;
  constexpr int kStageBytes = kOTileBytes + kWTileBytes;
  constexpr int kTmemCols = 2 * NT;
  constexpr int kHalf = NT / 2;  // columns of one epilogue warp
  static_assert(kHalf % 32 == 0, "an epilogue warp reads whole 32-column pieces");
  constexpr int kRound = kHalf >= 64 ? 64 : 32;  // columns an owner warp rounds before it stores row pieces
  constexpr int kRowBytes = kRound * 2, kPieces = kRowBytes / 16;
  const int n_tiles = p.hidden / NT;
  const int m_tiles = (p.n + kOBM - 1) / kOBM;
  const int tiles = m_tiles * n_tiles;
  const int kblocks = p.k / kOBK;
  constexpr bool kBf16 = !std::is_same<T, __half>::value;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kOEpiWarps);
    }
    sh_abort = 0;
    mbar_fence_init();
  }
  if (warp == kOMmaWarp) {
    tc::tmem_alloc(&tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int *abort_flag = &sh_abort;
  auto wait = [&](uint64_t *bar, uint32_t parity, int where) -> bool {
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    if (lane == 0 || warp >= kOEpiWarps) report_error(p.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PEER, blockIdx.x, where);
    atomicExch(&sh_abort, 1);
    return false;
  };
  // a flag that another GPU raises: true once it has reached this step
  auto wait_flag = [&](const int32_t *flag, int where) -> bool {
    if (*abort_flag) return false;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      if (ld_acquire_sys(flag) - p.step >= 0) return true;  // step numbers only grow (wrap-safe)
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > 2000000000ull) {
        report_error(p.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PEER, blockIdx.x, where);
        atomicExch(&sh_abort, 1);
        return false;
      }
      __nanosleep(100);
    }
  };

  if (warp == kOProducerWarp) {
    if (lane == 0) {
      int it = 0;  // k-blocks issued so far (all tiles)
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int m = t / n_tiles, j = t - m * n_tiles;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = wait(&empty[s], ((it / STAGES) & 1) ^ 1, 100);
          if (!ok) break;
          mbar_arrive_expect_tx(&full[s], kStageBytes);
          const uint32_t dst = base + s * kStageBytes;
          tma_load_2d(dst, &tmap_a, kb * kOBK, m * kOBM, &full[s]);
          tma_load_2d(dst + kOTileBytes, &tmap_w, kb * kOBK, j * NT, &full[s]);
        }
        if (!ok) break;
      }
      // drain: nothing may still be landing when the CTA retires
      for (int x = it > STAGES ? it - STAGES : 0; x < it; ++x) mbar_wait(&full[x % STAGES], (x / STAGES) & 1, 200000000ull);
    }
  } else if (warp == kOMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc(kBf16, false, false, kOBM, NT);
      int it = 0, nt = 0;  // k-blocks / tiles consumed so far
      for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++nt) {
        const int buf = nt & 1;
        if (!wait(&acc_empty[buf], ((nt >> 1) & 1) ^ 1, 200)) break;  // the epilogue has read this accumulator
        tc::fence_after_sync();
        const uint32_t d = tmem + buf * NT;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = wait(&full[s], (it / STAGES) & 1, 210);
          if (!ok) break;
          tc::fence_after_sync();
          const uint64_t a_desc = tc::desc_k_major(base + s * kStageBytes);
          const uint64_t b_desc = tc::desc_k_major(base + s * kStageBytes + kOTileBytes);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::mma_ss(d, a_desc + (uint64_t)((ks * 32) >> 4), b_desc + (uint64_t)((ks * 32) >> 4), idesc,
                       (kb > 0 || ks > 0) ? 1u : 0u);
          tc::commit(&empty[s]);
        }
        if (!ok) break;
        tc::commit(&acc_full[buf]);
      }
    }
  } else {
    // ================================================ epilogue: thread = token row; warps w and w + 4 own the
    // same 32 rows (TMEM lanes) and take the lower / upper half of the tile's columns
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int c_half = (warp >> 2) * kHalf;
    const size_t tile_bytes = (size_t)kOBM * NT * (p.stage16 ? 2 : 4);
    // the warp's tile for the rows it is about to store: 32 rows x kRowBytes, 16-byte pieces swizzled by row
    uint8_t *wtile = smem_raw + (base - smem_u32(smem_raw)) + STAGES * kStageBytes + warp * (32 * kRowBytes);
    auto swz = [](int row, int piece) { return kPieces == 8 ? (piece ^ (row & 7)) : (piece ^ ((row >> 1) & 3)); };
    const int32_t *arrive_own = p.arrive[p.rank];
    const int32_t *done_own = p.done[p.rank];
    const uint8_t *stage_own = p.stage[p.rank];
    // Tile t belongs to rank t mod world.  With an even grid a CTA therefore keeps one role for all its tiles
    // (they are a grid apart): the senders run ahead of the owners of the same tiles on the other ranks, so
    // that an owner seldom waits for a partial.  Measured and not kept: roles that alternate from tile to tile
    // (every owned tile then waits for its sender in lockstep, 8 % slower on 8192 rows), and completion flags
    // raised one tile late (the wait moves from the fence into the stores: the link is the limit).
    int nt = 0;
    bool alive = true;
    OTRACE_DECL
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++nt) {
      const int m = t / n_tiles, j = t - m * n_tiles;
      const int buf = nt & 1;
      const int tok = m * kOBM + r;
      const bool row_ok = tok < p.n;
      const int owner = t % p.world, slot = t / p.world;
      if (!wait(&acc_full[buf], (nt >> 1) & 1, 300 + warp)) {
        alive = false;
        break;
      }
      __syncwarp();
      tc::fence_after_sync();
      OTRACE(0)
      const uint32_t acc = tmem + lane_base + buf * NT + c_half;
      if (owner != p.rank) {
        // ---- the partial goes to the owner
        uint8_t *tile = p.stage[owner] + ((size_t)p.rank * p.slots + slot) * tile_bytes;
#pragma unroll 1
        for (int ch = 0; ch < kHalf / 32; ++ch) {
          uint32_t v[32];
          tc::tmem_ld32(acc + ch * 32, v);
          tc::tmem_wait_ld();
          if (row_ok) {
            if (p.stage16) {
              uint4 *dst = reinterpret_cast<uint4 *>(tile) + (size_t)((c_half + ch * 32) / 8) * kOBM + r;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                dst[(size_t)q * kOBM] =
                    make_uint4(pack2<T>(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                               pack2<T>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                               pack2<T>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                               pack2<T>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
            } else {
              float4 *dst = reinterpret_cast<float4 *>(tile) + (size_t)((c_half + ch * 32) / 4) * kOBM + r;
#pragma unroll
              for (int q = 0; q < 8; ++q)
                dst[(size_t)q * kOBM] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                    __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
            }
          }
        }
        OTRACE(1)
        // One release at system scope by one lane, after the warp has met, covers every lane's stores (a
        // fence per thread costs tens of microseconds with 256 threads' peer stores in flight).
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&acc_empty[buf]);
          st_release_sys(p.arrive[owner] + ((size_t)slot * p.world + p.rank) * kOFlagsPerTile + warp, p.step);
        }
        OTRACE(2)
      } else {
        // ---- the sum over the ranks, the residual, one rounding, the rows to every rank
        bool ok = true;
        if (lane < p.world && lane != p.rank)
          ok = wait_flag(arrive_own + ((size_t)slot * p.world + lane) * kOFlagsPerTile + warp, 400 + lane);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          alive = false;
          break;
        }
        OTRACE(3)
        const T *res = p.residual != nullptr
                           ? reinterpret_cast<const T *>(p.residual) + (size_t)tok * p.residual_stride + (size_t)j * NT + c_half
                           : nullptr;
        // A round is kRound columns (64, or 32 for the narrowest tile): the thread that owns a row rounds
        // them into the warp's shared-memory tile, then the warp stores whole row pieces - eight (four)
        // lanes per row, 128 (64) contiguous bytes - so that what crosses NVLink are full lines, not the
        // 16-byte fragments a thread-per-row store would make.
#pragma unroll 1
        for (int round = 0; round < kHalf / kRound; ++round) {
#pragma unroll 1
          for (int sub = 0; sub < kRound / 32; ++sub) {
            const int ch = round * (kRound / 32) + sub;
            uint32_t v[32];
            tc::tmem_ld32(acc + ch * 32, v);
            tc::tmem_wait_ld();
            float s[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = 0.f;
            if (row_ok) {
              for (int src = 0; src < p.world; ++src) {
                if (src == p.rank) {
#pragma unroll
                  for (int i = 0; i < 32; ++i) s[i] += __uint_as_float(v[i]);
                } else if (p.stage16) {
                  const uint4 *sp = reinterpret_cast<const uint4 *>(stage_own + ((size_t)src * p.slots + slot) * tile_bytes) +
                                    (size_t)((c_half + ch * 32) / 8) * kOBM + r;
                  uint4 x[4];
#pragma unroll
                  for (int q = 0; q < 4; ++q) x[q] = __ldcg(sp + (size_t)q * kOBM);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    const uint32_t w4[4] = {x[q].x, x[q].y, x[q].z, x[q].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 f = unpack2<T>(w4[e]);
                      s[8 * q + 2 * e] += f.x;
                      s[8 * q + 2 * e + 1] += f.y;
                    }
                  }
                } else {
                  const float4 *sp = reinterpret_cast<const float4 *>(stage_own + ((size_t)src * p.slots + slot) * tile_bytes) +
                                     (size_t)((c_half + ch * 32) / 4) * kOBM + r;
                  float4 x[8];
#pragma unroll
                  for (int q = 0; q < 8; ++q) x[q] = __ldcg(sp + (size_t)q * kOBM);
#pragma unroll
                  for (int q = 0; q < 8; ++q) {
                    s[4 * q] += x[q].x;
                    s[4 * q + 1] += x[q].y;
                    s[4 * q + 2] += x[q].z;
                    s[4 * q + 3] += x[q].w;
                  }
                }
              }
              if (res != nullptr) {
                const uint4 *rp4 = reinterpret_cast<const uint4 *>(res + ch * 32);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 rv = rp4[q];
                  const uint32_t w4[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack2<T>(w4[e]);
                    s[8 * q + 2 * e] += f.x;
                    s[8 * q + 2 * e + 1] += f.y;
                  }
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int piece = sub * 4 + q;
              *reinterpret_cast<uint4 *>(wtile + lane * kRowBytes + swz(lane, piece) * 16) =
                  make_uint4(pack2<T>(s[8 * q], s[8 * q + 1]), pack2<T>(s[8 * q + 2], s[8 * q + 3]),
                             pack2<T>(s[8 * q + 4], s[8 * q + 5]), pack2<T>(s[8 * q + 6], s[8 * q + 7]));
            }
          }
          __syncwarp();
          const size_t col0 = (size_t)j * NT + c_half + round * kRound;
#pragma unroll
          for (int i = 0; i < kPieces; ++i) {
            const int row = lane / kPieces + i * (32 / kPieces), piece = lane % kPieces;
            const int tok2 = m * kOBM + (warp & 3) * 32 + row;
            if (tok2 < p.n) {
              const uint4 o = *reinterpret_cast<const uint4 *>(wtile + row * kRowBytes + swz(row, piece) * 16);
              const size_t off = (size_t)tok2 * p.hidden + col0 + piece * 8;
              for (int d = 0; d < p.world; ++d) *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(p.out[d]) + off) = o;
            }
          }
          __syncwarp();
        }
        OTRACE(4)
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&acc_empty[buf]);
          if (p.world > 1) {
            __threadfence_system();  // once, then a plain flag store per rank
            for (int d = 0; d < p.world; ++d)
              if (d != p.rank)
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.done[d] + (size_t)t * kOFlagsPerTile + warp),
                             "r"(p.step)
                             : "memory");
          }
        }
        OTRACE(5)
      }
    }
    // ---- this rank's output is whole once the owners of the tiles this CTA computed have stored them
    if (alive && p.world > 1) {
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        if (t % p.world == p.rank) continue;
        bool ok = true;
        if (lane == 0) ok = wait_flag(done_own + (size_t)t * kOFlagsPerTile + warp, 500);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
    }
    OTRACE(6)
#ifdef PIEKV_OTRACE
    if (warp == 0 && lane == 0 && p.trace != nullptr) {
      tr[7] = nt;
      for (int i = 0; i < 8; ++i) p.trace[(size_t)blockIdx.x * 8 + i] = tr[i];
    }
#endif
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == kOMmaWarp) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

template <typename T, int NT, int STAGES>
int launch_oproj(const CUtensorMap &ta, const CUtensorMap &tw, const OprojParams &p, cudaStream_t st) {
  constexpr int kSmemBytes = STAGES * (kOTileBytes + NT * kOBK * 2) + 1024 + kOEpiWarps * 32 * (NT >= 128 ? 128 : 64);
  static unsigned char configured[kMaxDevices] = {0};
  if (int rc = opt_in_dynamic_smem(oproj_reduce_kernel<T, NT, STAGES>, kSmemBytes, configured,
                                   "oproj_allreduce: cudaFuncSetAttribute"))
    return rc;
  const long long tiles = (long long)((p.n + kOBM - 1) / kOBM) * (p.hidden / NT);
  const int sms = sm_count();
  PIEKV_REQUIRE(sms > 0, "oproj_allreduce: cannot read the multiprocessor count");
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  oproj_reduce_kernel<T, NT, STAGES><<<grid, kOThreads, kSmemBytes, st>>>(ta, tw, p);
  PIEKV_LAUNCH_CHECK("oproj_reduce_kernel");
  return 0;
}

// Columns per tile: the widest tile (an MMA instruction does more, the rows of `a` are staged less often)
// that still gives most of the SMs a tile; the few rows of a decode step get narrow tiles so that many CTAs
// share the pass over w.
int oproj_tile_cols(int n, int hidden) {
  const long long m_tiles = (n + kOBM - 1) / kOBM;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  if (hidden % 256 == 0 && m_tiles * (hidden / 256) >= sms) return 256;
  if (hidden % 128 == 0 && m_tiles * (hidden / 128) * 4 >= 3 * sms) return 128;
  return 64;
}

}  // namespace
}  // namespace piekv

#ifdef PIEKV_OTRACE
static long long *g_otrace = nullptr;
extern "C" void *piekv_oproj_trace(void) {
  if (g_otrace == nullptr) cudaMalloc(&g_otrace, 256 * 8 * sizeof(long long));
  return g_otrace;
}
#endif

extern "C" int32_t piekv_oproj_tile_cols(int32_t n, int32_t hidden) {
  if (n <= 0 || hidden <= 0 || hidden % 64 != 0) return 0;
  return piekv::oproj_tile_cols(n, hidden);
}

extern "C" int piekv_oproj_allreduce_sizes(int32_t n_max, int32_t hidden, int32_t world, int64_t *sizes) {
  using namespace piekv;
  PIEKV_REQUIRE(n_max > 0 && hidden > 0 && hidden % 64 == 0 && world >= 1 && world <= PIEKV_MAX_PEERS && sizes != nullptr,
                "oproj_allreduce_sizes: bad arguments");
  const int64_t m_tiles = (n_max + kOBM - 1) / kOBM;
  // the narrow tiling has the most tiles (flags); a rank's staging holds world * slots tiles of a tiling
  const int64_t tiles64 = m_tiles * (hidden / 64);
  const int64_t slots64 = (tiles64 + world - 1) / world;
  int64_t stage = 0;
  for (int nt = 64; nt <= 256; nt *= 2) {
    if (hidden % nt != 0) continue;
    const int64_t slots = (m_tiles * (hidden / nt) + world - 1) / world;
    const int64_t bytes = slots * world * (int64_t)kOBM * nt * 4;
    if (bytes > stage) stage = bytes;
  }
  sizes[0] = world > 1 ? stage : 0;                       // staging bytes per rank
  sizes[1] = slots64 * world * kOFlagsPerTile;            // arrival flag words per rank
  sizes[2] = tiles64 * kOFlagsPerTile;                    // completion flag words per rank
  return 0;
}

extern "C" int piekv_oproj_allreduce(const void *a, int64_t a_stride_n, const void *w_o, int64_t w_stride_n,
                                     const void *residual, int64_t residual_stride_n, int32_t n, int32_t k_local,
                                     int32_t hidden, int32_t dtype, const piekv_peer_reduce *peers, int32_t *err,
                                     void *stream) {
  using namespace piekv;
  PIEKV_REQUIRE(dtype == PIEKV_BF16 || dtype == PIEKV_F16, "oproj_allreduce: 16-bit types only (dtype %d)", dtype);
  PIEKV_REQUIRE(n >= 0 && k_local > 0 && k_local % kOBK == 0, "oproj_allreduce: k_local %d is not a multiple of %d",
                k_local, kOBK);
  PIEKV_REQUIRE(hidden > 0 && hidden % 64 == 0, "oproj_allreduce: hidden %d is not a multiple of 64", hidden);
  PIEKV_REQUIRE(peers != nullptr && peers->world >= 1 && peers->world <= PIEKV_MAX_PEERS && peers->rank >= 0 &&
                    peers->rank < peers->world,
                "oproj_allreduce: bad peer description");
  if (n == 0) return 0;
  PIEKV_REQUIRE(a && w_o, "oproj_allreduce: null pointer");
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_o) & 15) == 0 &&
                    (a_stride_n * 2) % 16 == 0 && (w_stride_n * 2) % 16 == 0 && a_stride_n >= k_local &&
                    w_stride_n >= k_local,
                "oproj_allreduce: a and w_o rows must be 16-byte aligned and at least k_local long");
  PIEKV_REQUIRE(residual == nullptr || ((reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
                                        (residual_stride_n * 2) % 16 == 0 && residual_stride_n >= hidden),
                "oproj_allreduce: residual rows must be 16-byte aligned and at least `hidden` long");
  const int nt = oproj_tile_cols(n, hidden);
  const int64_t m_tiles = (n + kOBM - 1) / kOBM;
  const int64_t tiles = m_tiles * (hidden / nt);
  const int64_t slots = (tiles + peers->world - 1) / peers->world;
  OprojParams p{};
  p.n = n;
  p.k = k_local;
  p.hidden = hidden;
  p.world = peers->world;
  p.rank = peers->rank;
  p.step = peers->step;
  p.slots = (int)slots;
  p.stage16 = (peers->flags & PIEKV_REDUCE_PARTIALS_16BIT) ? 1 : 0;
  p.residual = residual;
  p.residual_stride = residual_stride_n;
  p.err = err;
#ifdef PIEKV_OTRACE
  p.trace = reinterpret_cast<long long *>(piekv_oproj_trace());
#endif
  for (int r = 0; r < peers->world; ++r) {
    PIEKV_REQUIRE(peers->out[r] != nullptr && (reinterpret_cast<uintptr_t>(peers->out[r]) & 15) == 0,
                  "oproj_allreduce: out[%d] missing or not 16-byte aligned", r);
    p.out[r] = peers->out[r];
    if (peers->world > 1) {
      PIEKV_REQUIRE(peers->stage[r] != nullptr && peers->arrive[r] != nullptr && peers->done[r] != nullptr &&
                        (reinterpret_cast<uintptr_t>(peers->stage[r]) & 15) == 0,
                    "oproj_allreduce: staging or flags of rank %d missing", r);
      p.stage[r] = reinterpret_cast<uint8_t *>(peers->stage[r]);
      p.arrive[r] = peers->arrive[r];
      p.done[r] = peers->done[r];
    }
  }
  if (peers->world > 1) {
    PIEKV_REQUIRE(peers->stage_bytes >= slots * peers->world * (int64_t)kOBM * nt * (p.stage16 ? 2 : 4) &&
                      peers->arrive_words >= slots * peers->world * kOFlagsPerTile &&
                      peers->done_words >= tiles * kOFlagsPerTile,
                  "oproj_allreduce: staging or flag arrays too small for %d rows (see piekv_oproj_allreduce_sizes)", n);
  }
  CUtensorMap ta, tw;
  if (int rc = make_matrix_tensor_map(&ta, a, n, k_local, a_stride_n, dtype, kOBM, kOBK)) return rc;
  if (int rc = make_matrix_tensor_map(&tw, w_o, hidden, k_local, w_stride_n, dtype, nt, kOBK)) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == PIEKV_BF16) {
    if (nt == 256) return launch_oproj<__nv_bfloat16, 256, 4>(ta, tw, p, st);
    if (nt == 128) return launch_oproj<__nv_bfloat16, 128, 6>(ta, tw, p, st);
    return launch_oproj<__nv_bfloat16, 64, 8>(ta, tw, p, st);
  }
  if (nt == 256) return launch_oproj<__half, 256, 4>(ta, tw, p, st);
  if (nt == 128) return launch_oproj<__half, 128, 6>(ta, tw, p, st);
  return launch_oproj<__half, 64, 8>(ta, tw, p, st);
}
