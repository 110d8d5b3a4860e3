// 2:4 structured-sparse W8A8 GEMM for sm_100a:
//     out(M tokens, N) = epilogue( X(M,K) s8 * Wpruned(N,K)^T -> s32 )
// The pruned weight is the sparse A operand of tcgen05.mma.sp kind::i8 (128 weight rows per
// tile on the 128 tensor-memory lanes); a block of tokens is the dense B operand, so the
// accumulator tile is D[weight row, token] and the epilogue writes it transposed.
//
// Per 256-deep K block a stage of shared memory holds
//     A  128 rows x 128 B      compressed weights, 128-byte swizzle            (TMA)
//     E  2 x (128 rows x 16 B) metadata, 8 nibbles per 32 K, plain rows        (TMA, no swizzle)
//     B  2 x (block_t rows x 128 B) int8 activations, 128-byte swizzle         (TMA)
// The MMA thread copies E into tensor memory with two tcgen05.cp (128 lanes x 128 bits each =
// the metadata of two K=64 instructions) and issues four tcgen05.mma.sp per stage.  tcgen05.cp
// and tcgen05.mma issued by one thread execute in issue order, so one 8-column metadata slot
// in tensor memory is enough.  Roles, accumulator double-buffering and bounded waits are as in
// the dense kernel.
//
// CTA-pair variant (kG == 2, cta_group::2): a tile is 256 weight rows x block_t tokens; each
// CTA stages its own 128 weight rows (A and E) and HALF of the token tile, so the activation
// traffic into shared memory -- most of a stage -- is halved per CTA.  Loads are plain
// cp.async.bulk.tensor ... .cta_group::2 crediting the leader's barrier (no multicast); the
// leader issues tcgen05.cp / tcgen05.mma.sp for the pair and commits to both CTAs' barriers.
#include "common.cuh"
#include <cstdlib>

namespace hy3d {
namespace sparse {
namespace {

constexpr int kTileW = 128;          // weight rows per tile (tensor-memory lanes)
constexpr int kBlockK = 256;         // logical K per stage (four K=64 instructions)
constexpr int kABytes = kTileW * (kBlockK / 2);   // 16384: 128 rows x 128 B of compressed weights
constexpr int kEBytes = kTileW * (kBlockK / 8);   // 4096: two 128 x 16 B metadata tiles
constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 16;                         // four per 32-lane quarter of tensor memory
constexpr int kWarpsPerQuarter = kEpiWarps / 4;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;
constexpr int kSlabTokens = 32;                       // tokens per TMA store
constexpr int kSlabBytes = kSlabTokens * 64;          // 32 tokens x 32 columns x 2 B
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxBlockT = 240;      // 2 * 240 accumulator columns + 8 metadata columns <= 512

struct SparseArgs {
  const float* act_scale;
  const void* w_scale;
  const void* bias;
  void* out;
  int ws_dtype, bias_dtype, out_dtype, epilogue;
  int M, N, K;
  int block_t, stages, tma_store;
  int w_tiles, t_tiles, num_kb, last_ksteps;
};

struct __align__(16) SparseCtrl {
  float as[2][256];     // per-token activation scales of the current tile, per accumulator buffer
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
}

__device__ __forceinline__ void store_one(void* out, int out_dtype, int64_t idx, float v) {
  if (out_dtype == HY3D_BF16)
    reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
}

// kBf16 / kEpi select the output packing and the epilogue at compile time for the 16-bit
// outputs (raw int32 output runs the <false, LINEAR> instance's direct-store path).
template <int kG, bool kBf16, int kEpi>
__global__ void __launch_bounds__(kThreads, 1)
gemm_sparse_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_e,
                   const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_o,
                   const SparseArgs p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t smem_base = smem_u32(smem_raw);
  if (smem_base & 1023u) {   // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(&g_device_status, 0, static_cast<int>(kDevBadAlignment));
    return;
  }

  // One 128-byte-wide box of tokens; with a CTA pair each CTA stages half of the token tile.
  const uint32_t b_half = static_cast<uint32_t>(p.block_t / kG) * 128u;
  const uint32_t b_bytes = 2u * b_half;
  const uint32_t stage_bytes = kABytes + kEBytes + b_bytes;
  const uint32_t staging_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
  SparseCtrl* ctrl = reinterpret_cast<SparseCtrl*>(smem + static_cast<size_t>(p.stages) * stage_bytes +
                                                   kEpiWarps * kSlabBytes);
  volatile int* abort_flag = &ctrl->abort_flag;

  // Warp index through a shuffle: known warp-uniform to the compiler, so the producer and MMA
  // roles run as warp-uniform loops (all lanes wait, lane 0 issues) with their descriptors and
  // coordinates in uniform registers.
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.w_tiles * p.t_tiles;       // w_tiles counts 128*kG-row units
  const uint32_t cta_rank = kG == 2 ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const int first_tile = static_cast<int>(blockIdx.x) / kG;
  const int tile_step = static_cast<int>(gridDim.x) / kG;
  const int row_off = static_cast<int>(cta_rank) * kTileW;                 // this CTA's weight rows
  const int tok_off = static_cast<int>(cta_rank) * (p.block_t / kG);       // this CTA's share of B
  const uint32_t tmem_cols = 512;
  const uint32_t e_col = static_cast<uint32_t>(2 * p.block_t);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), kG * kEpiWarps);   // one arrival per epilogue warp
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_e);
    tma_prefetch_desc(&tm_x);
    if (p.tma_store) tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    if (kG == 2) {
      tmem_alloc_2cta(smem_u32(&ctrl->tmem_base), tmem_cols);
      tmem_relinquish_2cta();
    } else {
      tmem_alloc_1cta(smem_u32(&ctrl->tmem_base), tmem_cols);
      tmem_relinquish_1cta();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kG == 2) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer (all lanes walk the loop, lane 0 issues) ----------------
    {
      const bool issuer = lane == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        const int w0 = (tile % p.w_tiles) * (kTileW * kG) + row_off;
        const int t0 = (tile / p.w_tiles) * p.block_t + tok_off;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, kDevTimeoutEmpty);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + kABytes + kEBytes;
          if (!issuer) {
            // only lane 0 issues
          } else if (kG == 1) {
            mbar_arrive_expect_tx(full, stage_bytes);
            tma_load_2d(sa, &tm_w, full, kb * (kBlockK / 2), w0);
            tma_load_2d(sa + kABytes, &tm_e, full, kb * (kBlockK / 8), w0);
            tma_load_2d(sa + kABytes + kEBytes / 2, &tm_e, full, kb * (kBlockK / 8) + 16, w0);
            tma_load_2d(sb, &tm_x, full, kb * kBlockK, t0);
            tma_load_2d(sb + b_half, &tm_x, full, kb * kBlockK + 128, t0);
          } else {
            // Both CTAs credit their bytes to the leader's barrier; only the leader arrives.
            const uint32_t full_leader = map_to_cta(full, 0);
            if (leader) mbar_arrive_expect_tx(full, 2 * stage_bytes);
            tma_load_2d_pair(sa, &tm_w, full_leader, kb * (kBlockK / 2), w0);
            tma_load_2d_pair(sa + kABytes, &tm_e, full_leader, kb * (kBlockK / 8), w0);
            tma_load_2d_pair(sa + kABytes + kEBytes / 2, &tm_e, full_leader, kb * (kBlockK / 8) + 16, w0);
            tma_load_2d_pair(sb, &tm_x, full_leader, kb * kBlockK, t0);
            tma_load_2d_pair(sb + b_half, &tm_x, full_leader, kb * kBlockK + 128, t0);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread) ----------------
    if (leader) {
      const bool issuer = lane == 0;
      const uint32_t idesc = make_idesc_i8(kTileW * kG, static_cast<uint32_t>(p.block_t), true);
      const uint64_t desc128 = make_smem_desc(0, 1024, 128);
      const uint64_t desc_e = make_smem_desc(0, 128, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait(smem_u32(&ctrl->tmem_empty[buf]), acc_phase ^ 1, abort_flag,
                       kDevTimeoutTmemEmpty);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.block_t);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = mbar_wait<true>(smem_u32(&ctrl->full[stage]), phase, abort_flag, kDevTimeoutFull);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t se = sa + kABytes;
          const uint32_t sb = se + kEBytes;
          const uint64_t da = desc128 | static_cast<uint64_t>((sa & 0x3FFFFu) >> 4);
          const uint64_t db0 = desc128 | static_cast<uint64_t>((sb & 0x3FFFFu) >> 4);
          const uint64_t db1 = desc128 | static_cast<uint64_t>(((sb + b_half) & 0x3FFFFu) >> 4);
          // Metadata of the stage: two 128-lane x 128-bit copies = 8 columns = four K=64 steps.
          const uint64_t de0 = desc_e | static_cast<uint64_t>((se & 0x3FFFFu) >> 4);
          const uint64_t de1 = desc_e | static_cast<uint64_t>(((se + kEBytes / 2) & 0x3FFFFu) >> 4);
          if (issuer) {
          if (kG == 1) {
            tmem_cp_128x128b_1cta(tmem_base + e_col, de0);
            tmem_cp_128x128b_1cta(tmem_base + e_col + 4, de1);
          } else {
            tmem_cp_128x128b_2cta(tmem_base + e_col, de0);
            tmem_cp_128x128b_2cta(tmem_base + e_col + 4, de1);
          }
          const int nk = (kb == p.num_kb - 1) ? p.last_ksteps : 4;
          // Per K=64 instruction: 32 compressed bytes of A (+2 address units), 64 bytes of B
          // (+4; the second 128-byte box after two steps) and two metadata columns.
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k < nk) {
              const uint64_t dbk = k < 2 ? db0 + 4 * k : db1 + 4 * (k - 2);
              if (kG == 1)
                mma_sp_i8_1cta(d_tmem, da + 2 * k, dbk, tmem_base + e_col + 2 * k, idesc,
                               (kb | k) != 0 ? 1u : 0u);
              else
                mma_sp_i8_2cta(d_tmem, da + 2 * k, dbk, tmem_base + e_col + 2 * k, idesc,
                               (kb | k) != 0 ? 1u : 0u);
            }
          }
          if (kG == 1) tc_commit_1cta(smem_u32(&ctrl->empty[stage]));
          else tc_commit_2cta(smem_u32(&ctrl->empty[stage]), 3);
          }   // issuer
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (ok && issuer) {
          if (kG == 1) tc_commit_1cta(smem_u32(&ctrl->tmem_full[buf]));
          else tc_commit_2cta(smem_u32(&ctrl->tmem_full[buf]), 3);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;                   // tensor-memory lane quarter
    const int half = (warp - 2) >> 2;               // which of the warps sharing it
    const int row_in_tile = quarter * 32 + lane;    // weight row within the tile
    const int et = threadIdx.x - 64;
    constexpr bool geglu = kEpi == HY3D_EPI_GEGLU;
    constexpr bool gelu = kEpi == HY3D_EPI_GELU;
    constexpr int kOutDtype = kBf16 ? HY3D_BF16 : HY3D_F16;
    const int64_t ldo = geglu ? (p.N >> 1) : p.N;
    const uint32_t stage_buf = staging_base + static_cast<uint32_t>(warp - 2) * kSlabBytes;
    bool ok = true;
    int it = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int w0 = (tile % p.w_tiles) * (kTileW * kG) + row_off;
      const int t0 = (tile / p.w_tiles) * p.block_t;
      const int n = w0 + row_in_tile;
      const bool n_ok = n < p.N;
      float ws = 0.0f, bs = 0.0f;
      float sc_next = 0.0f;
      if (p.out_dtype != HY3D_S32) {
        if (p.tma_store) {
          // Each warp stages the 32 token scales of its own slab (fetched one slab ahead), so
          // the tile needs no CTA-wide barrier.
          const int t = t0 + half * kSlabTokens + lane;
          if (half * kSlabTokens < p.block_t && t < p.M) sc_next = p.act_scale[t];
        } else {
          for (int c = et; c < p.block_t; c += kEpiThreads)
            ctrl->as[buf][c] = (t0 + c) < p.M ? p.act_scale[t0 + c] : 0.0f;
        }
        if (n_ok) {
          ws = load_scalar(p.w_scale, p.ws_dtype, n);
          bs = p.bias ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
        }
      }
      if (!p.tma_store) epi_bar_sync();
      if (ok) ok = mbar_wait(smem_u32(&ctrl->tmem_full[buf]), acc_phase, abort_flag,
                             kDevTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * p.block_t);
      const float* asb = ctrl->as[buf];
      if (p.tma_store) {
        float* asw = &ctrl->as[0][0] + (warp - 2) * kSlabTokens;   // this warp's 32 scales
        // Slabs of 32 tokens; this thread owns output column n, the warp 32 adjacent columns,
        // so a slab is a 32 (tokens) x 64 B block of the output, staged with 64-byte swizzle.
        const int nslab = p.block_t / kSlabTokens;
        const uint32_t chunk = static_cast<uint32_t>(lane) >> 3;
        const uint32_t in_chunk = (static_cast<uint32_t>(lane) & 7u) * 2u;
        for (int s = half; s < nslab; s += kWarpsPerQuarter) {
          const int c0 = s * kSlabTokens;
          uint32_t r[32];
          const float sc = sc_next;
          {
            const int sn = s + kWarpsPerQuarter;
            const int t = t0 + sn * kSlabTokens + lane;
            sc_next = (sn < nslab && t < p.M) ? p.act_scale[t] : 0.0f;
          }
          __syncwarp();
          asw[lane] = sc;
          tmem_ld_x32(t_row + c0, r);
          tmem_ld_wait();
          __syncwarp();
          float y[32];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 a4 = *reinterpret_cast<const float4*>(asw + 4 * q);
            y[4 * q + 0] = fmaf(static_cast<float>(static_cast<int32_t>(r[4 * q + 0])), a4.x * ws, bs);
            y[4 * q + 1] = fmaf(static_cast<float>(static_cast<int32_t>(r[4 * q + 1])), a4.y * ws, bs);
            y[4 * q + 2] = fmaf(static_cast<float>(static_cast<int32_t>(r[4 * q + 2])), a4.z * ws, bs);
            y[4 * q + 3] = fmaf(static_cast<float>(static_cast<int32_t>(r[4 * q + 3])), a4.w * ws, bs);
          }
          if (gelu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = gelu_erf(y[j]);
          }
          if (geglu) {
            // Weight rows come in blocks of 32 = 16 value rows then their 16 gate rows: lanes
            // 0-15 hold the values, lanes 16-31 the matching gates of the same tokens.
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = y[j] * gelu_erf(__shfl_down_sync(0xffffffffu, y[j], 16));
          }
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          if (!geglu) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              // token rows j, j+1 of the slab (64 B each): 16-byte chunk c of row j sits at
              // c ^ ((j >> 1) & 3), the same for both rows of a pair; one conversion packs both.
              const uint32_t addr = stage_buf + static_cast<uint32_t>(j) * 64u +
                                    ((chunk ^ ((static_cast<uint32_t>(j) >> 1) & 3u)) << 4) + in_chunk;
              const uint32_t pr = pack2(y[j], y[j + 1], kOutDtype);
              const uint16_t lo = static_cast<uint16_t>(pr & 0xFFFFu);
              const uint16_t hi = static_cast<uint16_t>(pr >> 16);
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(lo) : "memory");
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr + 64u), "h"(hi) : "memory");
            }
          } else if (lane < 16) {
            // 16 output columns per token: plain 32-byte rows (the store's box is 32 B wide)
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const uint32_t addr = stage_buf + static_cast<uint32_t>(j) * 32u + static_cast<uint32_t>(lane) * 2u;
              const uint32_t pr = pack2(y[j], y[j + 1], kOutDtype);
              const uint16_t lo = static_cast<uint16_t>(pr & 0xFFFFu);
              const uint16_t hi = static_cast<uint16_t>(pr >> 16);
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(lo) : "memory");
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr + 32u), "h"(hi) : "memory");
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int out_col = geglu ? ((w0 + quarter * 32) >> 1) : (w0 + quarter * 32);
            const int out_row = t0 + c0;
            if (out_col < ldo && out_row < p.M) tma_store_2d(&tm_o, stage_buf, out_col * 2, out_row);
            tma_store_commit();
          }
        }
      } else {
        // GEGLU: weight rows come in blocks of 32 = 16 value rows then their 16 gate rows, so
        // lanes 0-15 hold values and lanes 16-31 the matching gates.
        const int64_t out_col = geglu ? ((w0 + quarter * 32) >> 1) + (lane & 15) : n;
        for (int c = 16 * half; c < p.block_t; c += 16 * kWarpsPerQuarter) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_x16(t_row + c, r);
          tmem_ld_wait();
          if (p.out_dtype == HY3D_S32) {
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int t = t0 + c + j;
                if (t < p.M)
                  reinterpret_cast<int32_t*>(p.out)[static_cast<int64_t>(t) * ldo + n] =
                      static_cast<int32_t>(r[j]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c + j;
              float y = fmaf(static_cast<float>(static_cast<int32_t>(r[j])), asb[c + j] * ws, bs);
              if (gelu) y = gelu_erf(y);
              if (geglu) {
                const float g = __shfl_down_sync(0xffffffffu, y, 16);
                y = y * gelu_erf(g);
                if (lane < 16 && n_ok && t < p.M)
                  store_one(p.out, p.out_dtype, static_cast<int64_t>(t) * ldo + out_col, y);
              } else if (n_ok && t < p.M) {
                store_one(p.out, p.out_dtype, static_cast<int64_t>(t) * ldo + out_col, y);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        // The accumulator buffer goes back to the leader's MMA warp (own CTA or the peer).
        if (kG == 1 || leader) mbar_arrive(smem_u32(&ctrl->tmem_empty[buf]));
        else mbar_arrive_cluster(smem_u32(&ctrl->tmem_empty[buf]), 0);
      }
    }
    if (p.tma_store && lane == 0) tma_store_wait_all<0>();
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  // Neither CTA of a pair may retire while the other can still touch its shared memory,
  // barriers or tensor memory.
  if (kG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (kG == 2) tmem_dealloc_2cta(tmem_base, tmem_cols);
    else tmem_dealloc_1cta(tmem_base, tmem_cols);
  }
}

}  // namespace


int gemm_sparse24(const int8_t* X, const float* act_scale, const int8_t* w_comp,
                  const uint32_t* w_meta, int64_t meta_ld, const void* w_scale, int ws_dtype,
                  const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                  int64_t K, int epilogue, int block_t, cudaStream_t stream) {
  if (out_dtype != HY3D_F16 && out_dtype != HY3D_BF16 && out_dtype != HY3D_S32) return HY3D_ERR_ARG;
  if (epilogue < HY3D_EPI_LINEAR || epilogue > HY3D_EPI_GEGLU) return HY3D_ERR_ARG;
  if (out_dtype == HY3D_S32 && epilogue != HY3D_EPI_LINEAR) return HY3D_ERR_ARG;
  if (ws_dtype < HY3D_F16 || ws_dtype > HY3D_F32) return HY3D_ERR_ARG;
  if (bias && (bias_dtype < HY3D_F16 || bias_dtype > HY3D_F32)) return HY3D_ERR_ARG;
  if (M < 0 || N <= 0 || K <= 0 || (K & 63) || (N & 15)) return HY3D_ERR_SHAPE;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return HY3D_ERR_SHAPE;
  if (epilogue == HY3D_EPI_GEGLU && (N & 31)) return HY3D_ERR_SHAPE;
  const int64_t kblocks = (K + kBlockK - 1) / kBlockK;
  if (meta_ld != 4 * ((K + 127) / 128)) return HY3D_ERR_SHAPE;   // rows padded to 128-deep K blocks
  if (M == 0) return HY3D_OK;
  if (!X || !w_comp || !w_meta || !out) return HY3D_ERR_ARG;
  if (out_dtype != HY3D_S32 && (!act_scale || !w_scale)) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(w_comp) |
       reinterpret_cast<uintptr_t>(w_meta) | reinterpret_cast<uintptr_t>(out)) & 15)
    return HY3D_ERR_SHAPE;

  if (block_t == 0) {
    // Token-tile width that minimises rounds x time per tile: rounds = ceil(tiles / SMs), a
    // tile costs its width plus a fixed overhead worth ~94 columns of MMA time (the same
    // model as the dense kernel; measured on B200 the widest tile wins whenever the grid is
    // full, the narrowest when the whole problem is a single round).
    const int sms = device_sm_count() > 0 ? device_sm_count() : 148;
    const int64_t w_tiles = (N + kTileW - 1) / kTileW;
    int64_t best = -1;
    for (int bt = 224; bt >= 128; bt -= 32) {
      const int64_t tiles = w_tiles * ((M + bt - 1) / bt);
      const int64_t cost = ((tiles + sms - 1) / sms) * (bt + 94);
      if (best < 0 || cost < best) { best = cost; block_t = bt; }
    }
    if (M < block_t) block_t = static_cast<int>((M + 31) / 32 * 32);
  }
  if (block_t < 16 || block_t > kMaxBlockT || (block_t & 15)) return HY3D_ERR_SHAPE;

  // CTA pairs (256 weight rows sharing one token tile) halve each CTA's activation traffic
  // into shared memory, which is what paces deep-K stages (measured: 8192^3 384 -> 273 us,
  // M=3072 K=5120 N=1280 21.3 -> 15.7 us); on short K the per-tile hand-offs of a pair cost
  // more than that saves, and a weight matrix that fills its last 256-row tile badly (N = 320)
  // wastes the second CTA; launch-bound problems (M = 924) are faster with single CTAs.
  int group = 1;
  {
    const int64_t padded = ((N + 2 * kTileW - 1) / (2 * kTileW)) * (2 * kTileW);
    if (K >= 1024 && M >= 2048 && (block_t & 31) == 0 && padded * 4 <= N * 5) group = 2;
#ifdef HY3D_TRACE
    if (const char* e = getenv("HY3D_SPARSE_CTA_GROUP")) group = atoi(e) == 2 ? 2 : 1;
#endif
    if (group == 2 && (block_t & 31)) group = 1;
  }

  SparseArgs p;
  p.act_scale = act_scale; p.w_scale = w_scale; p.bias = bias; p.out = out;
  p.ws_dtype = ws_dtype; p.bias_dtype = bias_dtype; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.block_t = block_t;
  p.w_tiles = static_cast<int>((N + kTileW * group - 1) / (kTileW * group));
  p.t_tiles = static_cast<int>((M + block_t - 1) / block_t);
  p.num_kb = static_cast<int>(kblocks);
  const int k_last = static_cast<int>(K - (kblocks - 1) * kBlockK);
  p.last_ksteps = (k_last + 63) / 64;
  const int stage_bytes = kABytes + kEBytes + (block_t / group) * kBlockK;
  p.tma_store = (out_dtype != HY3D_S32 && block_t % kSlabTokens == 0) ? 1 : 0;
  const int fixed = static_cast<int>(sizeof(SparseCtrl)) + kEpiWarps * kSlabBytes;
  int stages = (kSmemLimit - fixed) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return HY3D_ERR_SHAPE;
  p.stages = stages;
  // One CTA per SM: the kernel allocates all 512 tensor-memory columns, so a second
  // resident CTA would wait for them.  Keep the footprint above half an SM's shared memory.
  int smem_bytes = stages * stage_bytes + fixed;
  if (smem_bytes < 120 * 1024) smem_bytes = 120 * 1024;

  CUtensorMap tm_w, tm_e, tm_x, tm_o;
  int rc = encode_tmap_2d_u8(&tm_w, w_comp, static_cast<uint64_t>(K / 2), static_cast<uint64_t>(N),
                             static_cast<uint64_t>(K / 2), 128, kTileW, 128);
  if (rc != HY3D_OK) return rc;
  rc = encode_tmap_2d_u8(&tm_e, w_meta, static_cast<uint64_t>(meta_ld * 4), static_cast<uint64_t>(N),
                         static_cast<uint64_t>(meta_ld * 4), 16, kTileW, 0);
  if (rc != HY3D_OK) return rc;
  rc = encode_tmap_2d_u8(&tm_x, X, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), 128, static_cast<uint32_t>(block_t / group), 128);
  if (rc != HY3D_OK) return rc;

  if (p.tma_store) {
    // A warp's slab is 32 tokens x 32 weight rows = 64 output bytes per token, or 16 outputs =
    // 32 bytes per token after the GEGLU gate.
    const bool geglu = epilogue == HY3D_EPI_GEGLU;
    const uint64_t row_bytes = static_cast<uint64_t>(geglu ? N / 2 : N) * 2;
    rc = encode_tmap_2d_u8(&tm_o, out, row_bytes, static_cast<uint64_t>(M), row_bytes, geglu ? 32 : 64,
                           kSlabTokens, geglu ? 0 : 64);
    if (rc != HY3D_OK) return rc;
  } else {
    tm_o = tm_x;   // unused by the kernel
  }

  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const CUtensorMap, const SparseArgs);
#define HY3D_SPARSE_ROW(G)                                                                                     \
  {{gemm_sparse_kernel<G, false, HY3D_EPI_LINEAR>, gemm_sparse_kernel<G, false, HY3D_EPI_GELU>,              \
    gemm_sparse_kernel<G, false, HY3D_EPI_GEGLU>},                                                            \
   {gemm_sparse_kernel<G, true, HY3D_EPI_LINEAR>, gemm_sparse_kernel<G, true, HY3D_EPI_GELU>,                \
    gemm_sparse_kernel<G, true, HY3D_EPI_GEGLU>}}
  static const KernelFn kernels[2][2][3] = {HY3D_SPARSE_ROW(1), HY3D_SPARSE_ROW(2)};
#undef HY3D_SPARSE_ROW
  const KernelFn kernel = kernels[group - 1][out_dtype == HY3D_BF16 ? 1 : 0][epilogue];
  rc = ensure_max_smem(reinterpret_cast<const void*>(kernel), kSmemLimit);
  if (rc != HY3D_OK) return rc;
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  const int total_tiles = p.w_tiles * p.t_tiles;
  const int max_clusters = sms / group;
  const int clusters = total_tiles < max_clusters ? total_tiles : max_clusters;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(group * clusters));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(group);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1] = pdl_attribute();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kernel, tm_w, tm_e, tm_x, tm_o, p) != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace sparse

using sparse::gemm_sparse24;

}  // namespace hy3d
