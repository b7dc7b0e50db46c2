// bf16 contraction on the 5th-generation tensor cores (tcgen05), fp32 accumulators
// in tensor memory, operands staged in shared memory by TMA.
//
// One persistent CTA per SM, 384 threads in three warpgroups:
//   warp 0       TMA producer (one elected lane)
//   warp 1       tensor-memory allocation, MMA issue (one elected lane)
//   warps 2..3   no role (they fill the first warpgroup)
//   warps 4..11  epilogue: warp w reads the 32 tensor-memory lanes of quarter w % 4;
//                warps 4..7 take columns 0..127 of the tile, warps 8..11 columns 128..255
// The kernel starts with 168 registers per thread (three warps per scheduler share its 16K
// registers); after set-up the first warpgroup hands registers back (setmaxnreg.dec to 72) and the
// two epilogue warpgroups take them (setmaxnreg.inc to 216: 128*72 + 256*216 = 384*168), so that the
// fused epilogues keep a 32-column chunk, its second operand and their results in registers while the
// next chunk's tensor-memory read is in flight.
// A CTA walks output tiles of 128 x 256 (tile index = blockIdx.x + i * gridDim.x).
// Four 48 KB stages (A 128x64, B 256x64 bf16) are handed from the producer to the
// MMA lane through full/empty mbarriers; two 256-column accumulators in tensor
// memory let the epilogue of one tile overlap the main loop of the next.
//
// Operand layouts.  Either operand may be K-major (the contraction axis is
// contiguous in global memory) or MN-major (the M or N axis is contiguous).
// Both are loaded with the 128-byte swizzle:
//   K-major : tensor (K, rows, z), one box of 64(K) x rows -> rows of 128 B,
//             8-row groups 1024 B apart; the 16-wide K step of one MMA moves the
//             start address by 32 B.
//   MN-major: tensor (MN, K, z), boxes of 64(MN) x 64(K), one per 64 rows/cols ->
//             K-rows of 128 B, 8-row groups 1024 B apart, boxes 8192 B apart; the
//             16-wide K step of one MMA moves the start address by 2048 B.
// No TMA load here uses cluster multicast.
//
// Every wait is bounded: a lane that gives up writes a code to the status word,
// raises the CTA's abort flag and all roles leave their loops; tensor memory is
// released on every path.
#pragma once

#include <cuda.h>

#include "epilogues.cuh"
#include "gemm.cuh"

namespace clt {
namespace tc {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;  // 16 KB
constexpr int kBBytes = kBN * kBK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = kFirstEpiWarp * 32 + kEpiThreads;
constexpr int kRegsLean = 72, kRegsEpi = 216;  // per-thread register budgets after set-up
constexpr int kTmemCols = 512;
constexpr int kMaxColArrays = 4;
constexpr int kColBytes = 2 * kMaxColArrays * kBN * 4;  // staged per-column parameters, double-buffered
constexpr int kEpiStageBytes = kEpiWarps * epi::kStageBytes;  // per-warp staging of coalesced stores
constexpr int kSmemBytes =
    kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kColBytes + kEpiStageBytes;
constexpr long long kWaitCycles = 4000000000ll;  // about two seconds

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the barrier did not flip in time
// or another role of this CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      report_status(status, code);
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Asynchronous read of 32 accumulator columns of this warp's 32 lanes; the registers are valid only
// after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128, N = 256.
//   bits 4-5 accumulator format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format,
//   bit 15 A is MN-major, bit 16 B is MN-major, bits 17-22 N >> 3, bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t instr_desc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

struct Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Order of the tiles of one slab.  CTAs work on consecutive tiles at the same time, so the faster axis
// is the one along which tiles share the LARGER operand: with more rows than columns (A is the big
// operand) the column tiles of one row block are neighbours and A's row block is fetched from HBM
// once and found in L2 by the others; with more columns than rows it is the other way round.
__device__ __forceinline__ void tile_origin(int r, int m_tiles, int n_tiles, int& m0, int& n0) {
  if (m_tiles > n_tiles) {
    m0 = (r / n_tiles) * kBM;
    n0 = (r % n_tiles) * kBN;
  } else {
    m0 = (r % m_tiles) * kBM;
    n0 = (r / m_tiles) * kBN;
  }
}

template <class Epi, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, GemmGeom g,
               typename Epi::Params ep, int* status) {
  extern __shared__ uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (g.M + kBM - 1) / kBM;
  const int n_tiles = (g.N + kBN - 1) / kBN;
  const int tiles_per_slab = m_tiles * n_tiles;
  const int total_tiles = tiles_per_slab * g.nz;
  const int kb_per_seg = (g.Kseg + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bars->full[i]), 1);
      mbar_init(smem_u32(&bars->empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->tmem_full[i]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[i]), kEpiWarps);  // one arrival per epilogue warp
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Register hand-over between the warpgroups: all four warps of a warpgroup execute one and the same
  // instruction, and the roles branch below it so that each branch is compiled for its own budget.
  if (warp < kFirstEpiWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLean));
    if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
          const int z = slab_of_rank(g, tile / tiles_per_slab);
          const int r = tile % tiles_per_slab;
          int m0, n0;
          tile_origin(r, m_tiles, n_tiles, m0, n0);
          const int nseg = seg_count(g, z);
          for (int j = 0; j < nseg && alive; ++j) {
            int za, zb;
            seg_index(g, z, j, za, zb);
            for (int kb = 0; kb < kb_per_seg; ++kb) {
              if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, status, kTimeoutEmpty)) {
                alive = false;
                break;
              }
              const uint32_t full = smem_u32(&bars->full[stage]);
              mbar_expect_tx(full, kStageBytes);
              const uint32_t sa = smem_u32(smem + stage * kStageBytes);
              const uint32_t sb = sa + kABytes;
              const int k0 = kb * kBK;
              if (A_MN) {
  #pragma unroll
                for (int i = 0; i < kBM / 64; ++i) tma_load_3d(sa + i * 8192, &mapA, full, m0 + 64 * i, k0, za);
              } else {
                tma_load_3d(sa, &mapA, full, k0, m0, za);
              }
              if (B_MN) {
  #pragma unroll
                for (int i = 0; i < kBN / 64; ++i) tma_load_3d(sb + i * 8192, &mapB, full, n0 + 64 * i, k0, zb);
              } else {
                tma_load_3d(sb, &mapB, full, k0, n0, zb);
              }
              if (++stage == kStages) stage = 0, phase ^= 1;
            }
          }
        }
        if (!alive) {
          // let copies that are still in flight land before the CTA's shared memory goes away
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------ MMA issuer --------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc = instr_desc(A_MN, B_MN);
        int stage = 0;
        uint32_t phase = 0;
        uint32_t acc_phase[2] = {0, 0};
        int it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++it) {
          const int buf = it & 1;
          const int z = slab_of_rank(g, tile / tiles_per_slab);
          const int nkb = seg_count(g, z) * kb_per_seg;
          if (!mbar_wait(smem_u32(&bars->tmem_empty[buf]), acc_phase[buf] ^ 1, abort_flag, status, kTimeoutTmemEmpty))
            break;
          acc_phase[buf] ^= 1;
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * kBN;
          for (int kb = 0; kb < nkb; ++kb) {
            if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, status, kTimeoutFull)) {
              alive = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * kStageBytes);
            const uint32_t sb = sa + kABytes;
  #pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              const uint64_t da = A_MN ? smem_desc(sa + k * 2048, 8192, 1024) : smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? smem_desc(sb + k * 2048, 8192, 1024) : smem_desc(sb + k * 32, 16, 1024);
              umma_bf16(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&bars->empty[stage]));  // frees the stage once these MMAs have read it
            if (++stage == kStages) stage = 0, phase ^= 1;
          }
          if (alive) umma_commit(smem_u32(&bars->tmem_full[buf]));
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpi));
    static_assert(Epi::kColArrays <= kMaxColArrays, "too many per-column parameter arrays");
    float* colp_base = reinterpret_cast<float*>(smem + kStages * kStageBytes + 256);
    unsigned char* stage = smem + kStages * kStageBytes + 256 + kColBytes + (warp - kFirstEpiWarp) * epi::kStageBytes;
    const int et = threadIdx.x - kFirstEpiWarp * 32;  // 0..255 among the epilogue threads
    const int quarter = warp & 3;                     // tensor-memory lanes 32*quarter .. +31
    const int half = (warp - kFirstEpiWarp) >> 2;     // which 128 columns of the tile
    typename Epi::State st;
    Epi::init(st);
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const int z = slab_of_rank(g, tile / tiles_per_slab);
      const int r = tile % tiles_per_slab;
      int m0, n0;
      tile_origin(r, m_tiles, n_tiles, m0, n0);
      float* colp = colp_base + buf * (kMaxColArrays * kBN);
      // stage this tile's per-column parameters while its main loop is still running
#pragma unroll
      for (int a = 0; a < Epi::kColArrays; ++a)
        colp[a * kBN + et] = (n0 + et < g.N) ? Epi::col_value(ep, a, z, n0 + et, g.N) : 0.f;
      int bad = 0;
      if (lane == 0)
        bad = mbar_wait(smem_u32(&bars->tmem_full[buf]), acc_phase[buf], abort_flag, status, kTimeoutTmemFull) ? 0 : 1;
      // one barrier over the epilogue threads: publishes the staged columns and makes the
      // give-up decision uniform, so no warp is left behind at a later barrier
      int any_bad;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.b32 p, %1, 0;\n\t"
          "bar.red.or.pred q, 1, %2, p;\n\t"
          "selp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(any_bad)
          : "r"(bad), "n"(kEpiThreads)
          : "memory");
      if (any_bad) break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < g.M;
      // the warp's 4 chunks of 32 columns
      constexpr int kChunks = kBN / 64;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kBN + 32 * half * kChunks);
      const int nbase = n0 + 32 * half * kChunks;
      // Neither loop below is unrolled further: an epilogue body is several thousand instructions, and
      // four copies of it per tile overflow the instruction cache.
      if constexpr (Epi::kPrefetch) {
        // two chunks per iteration; the read of the next chunk is in flight while one is processed
        static_assert(kChunks % 2 == 0, "chunks are taken in pairs");
        uint32_t ra[32], rb[32];
        if (nbase < g.N) tmem_ld32_issue(taddr0, ra);
#pragma unroll 1
        for (int cc = 0; cc < kChunks; cc += 2) {
          const int n = nbase + 32 * cc;
          if (n >= g.N) break;
          tmem_ld_wait();
          const bool second = n + 32 < g.N;
          if (second) tmem_ld32_issue(taddr0 + 32 * (cc + 1), rb);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
          Epi::template apply<kBN>(ep, st, z, row, row_ok, n, g.M, g.N, v, colp + 32 * (half * kChunks + cc), stage);
          if (!second) break;
          tmem_ld_wait();
          if (cc + 2 < kChunks && n + 64 < g.N) tmem_ld32_issue(taddr0 + 32 * (cc + 2), ra);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rb[i]);
          Epi::template apply<kBN>(ep, st, z, row, row_ok, n + 32, g.M, g.N, v, colp + 32 * (half * kChunks + cc + 1),
                                   stage);
        }
      } else {
#pragma unroll 1
        for (int cc = 0; cc < kChunks; ++cc) {
          const int n = nbase + 32 * cc;
          if (n >= g.N) break;
          uint32_t ra[32];
          tmem_ld32_issue(taddr0 + 32 * cc, ra);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
          Epi::template apply<kBN>(ep, st, z, row, row_ok, n, g.M, g.N, v, colp + 32 * (half * kChunks + cc), stage);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[buf]));
    }
    Epi::finish(ep, st);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ----------------------------------------------------------------------
struct TcOperand {
  const void* ptr;      // bf16
  int mn_major;         // 0: rows are the M (or N) axis and K is contiguous; 1: rows are K and M (or N) is contiguous
  long long inner;      // length of the contiguous axis
  long long rows;       // number of rows of one matrix
  long long row_stride; // elements between rows
  long long z_count;    // stacked matrices
  long long z_stride;   // elements between matrices
};

int encode_operand_map(CUtensorMap* map, const TcOperand& o, int tile_rows_if_k_major);

template <class Epi, bool A_MN, bool B_MN>
int launch_gemm_tc_impl(const GemmGeom& g, const TcOperand& a, const TcOperand& b, const typename Epi::Params& ep,
                        int* status, int num_sms, cudaStream_t stream) {
  CUtensorMap mapA, mapB;
  if (int rc = encode_operand_map(&mapA, a, kBM)) return rc;
  if (int rc = encode_operand_map(&mapB, b, kBN)) return rc;
  auto kern = gemm_tc_kernel<Epi, A_MN, B_MN>;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    CLT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set = true;
  }
  const long long m_tiles = (g.M + kBM - 1) / kBM, n_tiles = (g.N + kBN - 1) / kBN;
  const long long total = m_tiles * n_tiles * g.nz;
  if (total <= 0) return 0;
  CLT_CHECK_ARG(total < (1ll << 31), "gemm_tc: too many tiles");
  const int grid = (int)(total < num_sms ? total : num_sms);
  kern<<<grid, kThreads, kSmemBytes, stream>>>(mapA, mapB, g, ep, status);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <class Epi>
int launch_gemm_tc(const GemmGeom& g, const TcOperand& a, const TcOperand& b, const typename Epi::Params& ep,
                   int* status, int num_sms, cudaStream_t stream) {
  if (a.mn_major) {
    if (b.mn_major) return launch_gemm_tc_impl<Epi, true, true>(g, a, b, ep, status, num_sms, stream);
    return launch_gemm_tc_impl<Epi, true, false>(g, a, b, ep, status, num_sms, stream);
  }
  if (b.mn_major) return launch_gemm_tc_impl<Epi, false, true>(g, a, b, ep, status, num_sms, stream);
  return launch_gemm_tc_impl<Epi, false, false>(g, a, b, ep, status, num_sms, stream);
}

}  // namespace tc
}  // namespace clt
