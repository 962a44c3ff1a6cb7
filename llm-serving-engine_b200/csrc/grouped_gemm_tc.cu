// bfloat16 products of sorted rows with the weights of the expert each row belongs to, on the
// 5th-generation tensor cores:
//   out[r, n] = scale[r] * sum_k a[r, k] * w[e(r), n, k]        float32 accumulation and output
//
// The rows of `a` lie sorted by expert; a *tile* is up to 128 consecutive rows of one expert
// (tile_batch, tile_row0 as lse_moe_sort leaves them with tiles of 128 rows). One block computes
// 256 output features of one tile: as in the few-rows product the weights are the M operand of
// tcgen05.mma (two instructions of M = 128 per k step, which share the rows' tile) and the tile's
// rows its N dimension (128), both K-major in global memory, so TMA brings a [256, 64] tile of
// weights and a [128, 64] tile of rows per stage into 128-byte-swizzled shared memory (the weights
// of all experts are one [E * N, K] matrix to TMA; the rows one [rows, K] matrix): 48 KB feed
// 2 x 128 x 128 x 64 multiply-adds, which is what keeps the tiles' traffic from L2 below what the
// tensor cores could consume. One thread runs the TMA pipeline, one issues the MMAs with two
// accumulators [128 x 128] in tensor memory, four warps read them back and write out[r, n] with
// n across lanes. Rows of the tile that lie past the expert's range (they are the next expert's,
// or past the end) are computed and not stored; so are features past the expert's N. Two blocks
// share an SM (two stages and 256 columns of tensor memory each): one block's set-up and
// epilogue run under the other's MMAs (measured: 862 TFLOP/s against 643 with one block of four
// stages, on 4096 rows over 8 experts of 4096 x 2048).
//
// Every wait on an mbarrier is bounded: on expiry the block records an error code in *error_flag
// and leaves through the normal teardown (tensor memory is released).
#include "kernels.h"
#include "tma_util.cuh"

namespace lse {
namespace gtc {

constexpr int BM = 256;  // output features per block: two MMAs of M = 128
constexpr int BT = 128;  // rows per tile (MMA N)
constexpr int BK = 64;   // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 2;

using namespace tma;

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Params {
  int N, K, chunks;  // features per expert; k stages of 64
  float* out;        // [rows, N]
  const float* scale;   // per choice, or null
  const int* perm;      // sorted row -> choice (read with scale only)
  const int* offsets;   // [E + 1]
  const int* tile_batch;
  const int* tile_row0;
  const int* num_tiles;
  int* error_flag;
};

__global__ void __launch_bounds__(192)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                    const Params p) {
  constexpr uint32_t W_BYTES = BM * BK * 2, A_BYTES = BT * BK * 2;
  constexpr uint32_t TMEM_COLS = 2 * BT;  // one accumulator per half of the features
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* w_tiles = base;
  unsigned char* a_tiles = base + STAGES * W_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(a_tiles + STAGES * A_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;  // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  __shared__ volatile int failed;
  __shared__ volatile int issued;  // stages the producer has requested from TMA
  __shared__ float row_scale[BT];  // what each row of the tile is multiplied by

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the tile list is written by the sorting kernel before this one: read it after the wait
  pdl_wait();
  if ((int)blockIdx.y >= *p.num_tiles) return;  // the whole block leaves: nothing was set up yet
  const int expert = p.tile_batch[blockIdx.y];
  const int row0 = p.tile_row0[blockIdx.y];
  const int rows = min(BT, p.offsets[expert + 1] - row0);
  const int n0 = blockIdx.x * BM;
  const int units = p.chunks;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    failed = 0;
    issued = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {  // one warp allocates tensor memory for the block
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: one (weights, rows) stage per unit
      for (int it = 0; it < units && !failed; ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
          failed = 1;
          break;
        }
        mbar_expect_tx(&full[s], W_BYTES + A_BYTES);
        tma_load_2d(w_tiles + s * W_BYTES, &map_w, &full[s], it * BK, expert * p.N + n0);
        tma_load_2d(a_tiles + s * A_BYTES, &map_a, &full[s], it * BK, row0);
        issued = it + 1;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(128, BT);
      bool ok = true;
      for (int it = 0; it < units && !failed; ++it) {
        const int s = it % STAGES;
        ok = mbar_wait(&full[s], (it / STAGES) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc_sw128(smem_u32(w_tiles + s * W_BYTES));
        const uint64_t db = smem_desc_sw128(smem_u32(a_tiles + s * A_BYTES));
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // 16 k-elements = 32 bytes further along the swizzled row: +2 in the address field
          umma(tmem_base, da + 2 * kk, db + 2 * kk, idesc, (it > 0 || kk > 0) ? 1u : 0u);
          // features 128 .. 255 of the tile: 128 rows of 128 bytes further on, in the next columns
          umma(tmem_base + BT, da + (128 * 128 >> 4) + 2 * kk, db + 2 * kk, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);  // arrives when the MMAs that read this stage are done
      }
      if (!ok) failed = 3;
      else umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    // ---- epilogue: warp w may read TMEM lanes 32*(w%4) .. +31, i.e. accumulator rows of that quarter
    const int quarter = warp & 3;
    // the rows' factors, fetched while the main loop runs (two dependent loads each)
    for (int t = (warp - 2) * 32 + lane; t < BT; t += 128)
      row_scale[t] = (p.scale && t < rows) ? p.scale[p.perm[row0 + t]] : 1.f;
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
    if (!mbar_wait(acc_full, 0)) {
      failed = 4;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int half_t0 = 0; half_t0 < 2 * BT; half_t0 += 16) {
        const int half = half_t0 / BT, t0 = half_t0 - half * BT;
        if (t0 >= rows) continue;
        const int n = n0 + half * 128 + quarter * 32 + lane;
        uint32_t v[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * BT + t0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,"
            "%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
              "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + j;
            if (t >= rows) break;
            p.out[(size_t)(row0 + t) * p.N + n] = __uint_as_float(v[j]) * row_scale[t];
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // every role is done; `failed` is final
  if (threadIdx.x == 0 && failed != 0) {
    if (p.error_flag) atomicExch(p.error_flag, 200 + failed);
    // copies that were requested must land before the block's shared memory is given up
    for (int c = max(0, issued - STAGES); c < issued; ++c)
      if (!mbar_wait(&full[c % STAGES], (c / STAGES) & 1)) break;
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

}  // namespace gtc
}  // namespace lse

using namespace lse;

extern "C" int lse_expert_linear_tc_tile_rows(void) { return gtc::BT; }

extern "C" int lse_expert_linear_tc(const void* a, const void* w, float* out, int rows, int E, int N,
                                    int K, const float* scale, const int* perm, const int* offsets,
                                    const int* tile_batch, const int* tile_row0, const int* num_tiles,
                                    int max_tiles, int* error_flag, cudaStream_t stream) {
  if (rows <= 0 || N <= 0 || max_tiles <= 0) return LSE_OK;
  if (K <= 0 || K % 8 || E <= 0 || !offsets || !tile_batch || !tile_row0 || !num_tiles) return LSE_BAD_ARGUMENT;
  if (scale && !perm) return LSE_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) return LSE_BAD_ARGUMENT;
  if (max_tiles > 65535) return LSE_BAD_ARGUMENT;
  CUtensorMap mw, ma;
  if (!tma::make_map_bf16(&mw, w, (long long)E * N, K, K, gtc::BM) ||
      !tma::make_map_bf16(&ma, a, rows, K, K, gtc::BT))
    return LSE_LAUNCH_FAILED;
  gtc::Params p;
  p.N = N; p.K = K; p.chunks = (K + gtc::BK - 1) / gtc::BK;
  p.out = out; p.scale = scale; p.perm = perm; p.offsets = offsets;
  p.tile_batch = tile_batch; p.tile_row0 = tile_row0; p.num_tiles = num_tiles; p.error_flag = error_flag;
  constexpr int smem = gtc::STAGES * (gtc::BM + gtc::BT) * gtc::BK * 2 + (2 * gtc::STAGES + 1) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gtc::grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return LSE_LAUNCH_FAILED;
    configured = true;
  }
  dim3 grid((N + gtc::BM - 1) / gtc::BM, max_tiles);
  return lse::launch(gtc::grouped_gemm_kernel, grid, 192, smem, stream, mw, ma, p) == cudaSuccess
             ? LSE_OK
             : LSE_LAUNCH_FAILED;
}
