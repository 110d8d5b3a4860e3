// Dense W8A8 GEMM for sm_100a: out = epilogue( A(M,K) s8 * B(N,K)^T s8 -> s32 ).
//
// One persistent CTA per SM walks 128 x block_n output tiles.  Roles by warp:
//   warp 0      TMA producer: A (128 x 128 B) and B (block_n x 128 B) boxes, 128-byte swizzle,
//               into a ring of shared-memory stages, signalled through "full" mbarriers.  Where
//               the CTA keeps one tile column and its B tile fits, B is loaded once and stays
//               resident; only A streams.
//   warp 1      owns tensor memory; issues tcgen05.mma kind::i8 (128 x block_n x 32 per
//               instruction, int32 accumulators in tensor memory) and commits each stage back
//               to its "empty" mbarrier.
//               Both of these run as warp-uniform loops: all lanes wait and count, lane 0 issues.
//   warps 2-17  epilogue, four warps per 32-lane quarter of tensor memory, alternating over
//               32-column slabs: tcgen05.ld, acc * (act_scale[m] * w_scale[n]) + bias[n],
//               optional GELU / GEGLU, pack to bf16 / fp16 into a 64-byte-swizzled staging
//               buffer, one TMA store per slab (rows and columns outside the matrix are
//               clipped by the tensor map).  Raw int32 output and tile widths that are not a
//               multiple of the slab use plain 16-byte stores instead.
// Two accumulator buffers in tensor memory let the epilogue of tile i overlap the MMAs of
// tile i+1.  Every wait is bounded; a wait that runs out records a code in the device
// status word and all roles fall through to the common teardown.
#include "common.cuh"
#include <cstdlib>

namespace hy3d {
// Host-side helpers implemented in capi.cu.
int encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                      uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, int swizzle_bytes);
int device_sm_count();
int current_device();
// Raises a kernel's dynamic shared-memory limit once per (device, kernel); thread-safe.
int ensure_max_smem(const void* kernel, int bytes);

namespace dense {
namespace {

constexpr int kTileM = 128;
constexpr int kBlockKBytes = 128;   // one 128-byte swizzle row of int8 = 128 K elements
constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 16;                       // four per 32-lane quarter of tensor memory
constexpr int kWarpsPerQuarter = kEpiWarps / 4;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;
constexpr int kSlabCols = 32;                       // output columns per TMA store
constexpr int kSlabBytes = 32 * kSlabCols * 2;      // 32 rows x 64 B
constexpr int kSmemLimit = 227 * 1024;

struct DenseArgs {
  const float* act_scale;
  const void* w_scale;
  const void* bias;
  void* out;
  int ws_dtype, bias_dtype, out_dtype, epilogue;
  int M, N, K;
  int block_n, stages, acc_cols, tma_store, store_bufs;
  int splits;        // split-K: the launch walks total_tiles x splits (tile, K range) units ...
  int kb_per_split;  // ... of this many pipeline stages each, writing raw int32 partials ...
  int64_t split_stride;   // ... `split_stride` elements apart behind `out`
  int m_rows_pad;         // rows of one partial matrix (M rounded up to whole tiles)
  int b_resident;  // the CTA's B tile (all K blocks) is loaded once and stays in shared memory
  int m_tiles, n_tiles, num_kb, last_ksteps, n_fastest;
  int atoms;   // 128-byte K blocks per pipeline stage (1 or 2)
  int debug;   // knock-out switches of -DHY3D_TRACE / -DHY3D_KO diagnostic builds (always 0 in the shipped library)
};

struct __align__(16) DenseCtrl {
  float ws[256];        // per-column weight scales of the current tile columns
  float bs[256];        // per-column bias
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t b_full;      // resident-B mode: the whole B tile has landed
  uint32_t tmem_base;
  int abort_flag;
};

// Timeline records of two epilogue warps (the first and the last) in -DHY3D_TRACE builds.
#ifdef HY3D_TRACE
#define HY3D_EPI_TRACE(ev, arg)                                              \
  do {                                                                       \
    if (threadIdx.x == 64) HY3D_TRACE_EVENT(2, tr, ev, arg);                 \
    else if (threadIdx.x == kThreads - 32) HY3D_TRACE_EVENT(0, tr, ev, arg); \
  } while (0)
#else
#define HY3D_EPI_TRACE(ev, arg) ((void)0)
#endif

__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2t(float a, float b) {
  if (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 32 accumulator columns of one row -> 32 outputs packed in 16 words.
template <bool kBf16, int kEpi>
__device__ __forceinline__ void slab_math(const uint32_t (&r)[32], float as, const float* wsb,
                                          const float* bsb, uint32_t (&packed)[16]) {
  // Packed fp32x2 instructions: two IEEE multiplies / fused multiply-adds per issue slot, the
  // same bits as the scalar forms.
  const float2 as2 = make_float2(as, as);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 w4 = *reinterpret_cast<const float4*>(wsb + 4 * q);
    const float4 b4 = *reinterpret_cast<const float4*>(bsb + 4 * q);
    const float2 s01 = __fmul2_rn(as2, make_float2(w4.x, w4.y));
    const float2 s23 = __fmul2_rn(as2, make_float2(w4.z, w4.w));
    const float2 a01 = make_float2(static_cast<float>(static_cast<int32_t>(r[4 * q + 0])),
                                   static_cast<float>(static_cast<int32_t>(r[4 * q + 1])));
    const float2 a23 = make_float2(static_cast<float>(static_cast<int32_t>(r[4 * q + 2])),
                                   static_cast<float>(static_cast<int32_t>(r[4 * q + 3])));
    const float2 y01 = __ffma2_rn(a01, s01, make_float2(b4.x, b4.y));
    const float2 y23 = __ffma2_rn(a23, s23, make_float2(b4.z, b4.w));
    float y0 = y01.x, y1 = y01.y, y2 = y23.x, y3 = y23.y;
    if (kEpi == HY3D_EPI_GELU) {
      y0 = gelu_erf(y0); y1 = gelu_erf(y1); y2 = gelu_erf(y2); y3 = gelu_erf(y3);
    }
    packed[2 * q] = pack2t<kBf16>(y0, y1);
    packed[2 * q + 1] = pack2t<kBf16>(y2, y3);
  }
}

// 64 accumulator columns = two blocks of (16 value | 16 gate) -> 32 outputs in 16 words.
template <bool kBf16>
__device__ __forceinline__ void slab_math_geglu(const uint32_t (&rv)[16], const uint32_t (&rg)[16],
                                                float as, const float* wsb, const float* bsb,
                                                uint32_t* packed8) {
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    float y[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float v = fmaf(static_cast<float>(static_cast<int32_t>(rv[j + u])), as * wsb[j + u],
                           bsb[j + u]);
      const float g = fmaf(static_cast<float>(static_cast<int32_t>(rg[j + u])),
                           as * wsb[16 + j + u], bsb[16 + j + u]);
      y[u] = v * gelu_erf(g);
    }
    packed8[j >> 1] = pack2t<kBf16>(y[0], y[1]);
  }
}

// Writes one packed 32 x 32 slab row into the warp's staging buffer (64-byte swizzle: 16-byte
// chunk c of row r sits at c ^ ((r >> 1) & 3)) and lets lane 0 issue the TMA store.
// `pending_ok` = number of earlier bulk groups of this warp that may still be reading
// shared memory (1 with two staging buffers, 0 with one).
__device__ __forceinline__ void slab_store(const uint32_t (&packed)[16], uint32_t buf_addr, int lane,
                                           int pending_ok, const CUtensorMap* tm_o, int x_bytes,
                                           int y_row, bool in_range) {
  if (lane == 0) {
    if (pending_ok) tma_store_wait_read<1>(); else tma_store_wait_read<0>();
  }
  __syncwarp();
  const uint32_t row_addr = buf_addr + static_cast<uint32_t>(lane) * 64u;
  const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll
  for (uint32_t c = 0; c < 4; ++c)
    st_shared_v4(row_addr + ((c ^ sw) << 4), packed[4 * c], packed[4 * c + 1], packed[4 * c + 2],
                 packed[4 * c + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (in_range) tma_store_2d(tm_o, buf_addr, x_bytes, y_row);
    tma_store_commit();
  }
}

template <bool kBf16, int kEpi, int kG, int kAtoms>
__global__ void __launch_bounds__(kThreads, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_o, const DenseArgs p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t smem_base = smem_u32(smem_raw);
  if (smem_base & 1023u) {   // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(&g_device_status, 0, static_cast<int>(kDevBadAlignment));
    return;
  }

  const uint32_t a_bytes = kTileM * kBlockKBytes;
  // With a CTA pair (kG == 2) each CTA stages its own 128 rows of A and half of the B tile.
  const uint32_t b_bytes = static_cast<uint32_t>(p.block_n / kG) * kBlockKBytes;
  // A stage holds kAtoms 128-byte-wide K blocks of each operand: [A0][A1..][B0][B1..].
  // Resident-B mode (one CTA per tile, one K block per stage): a stage holds A only, and the
  // CTA's B tile -- it keeps one tile column for the whole launch -- sits behind the ring.
  const bool b_res = kG == 1 && kAtoms == 1 && p.b_resident;
  const uint32_t stage_bytes = b_res ? a_bytes : static_cast<uint32_t>(kAtoms) * (a_bytes + b_bytes);
  const uint32_t b_res_base = smem_base + static_cast<uint32_t>(p.stages) * stage_bytes;
  const uint32_t b_res_bytes = b_res ? static_cast<uint32_t>(p.num_kb) * b_bytes : 0u;
  const uint32_t staging_base = b_res_base + b_res_bytes;
  DenseCtrl* ctrl = reinterpret_cast<DenseCtrl*>(smem + (staging_base - smem_base) +
                                                 kEpiWarps * p.store_bufs * kSlabBytes);
  volatile int* abort_flag = &ctrl->abort_flag;

  // The warp index comes through a shuffle so that the compiler knows it is the same for the
  // whole warp: the producer and MMA roles below then run as warp-uniform loops (all 32 lanes
  // wait and count, one lane issues), and their descriptors, coordinates and barrier
  // addresses can live in uniform registers instead of being converted for every issue.
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;     // m_tiles counts 128*kG-row units
  // Split-K launches walk (tile, K range) units: unit u = split * total_tiles + tile.
  const int total_units = total_tiles * p.splits;
  const uint32_t cta_rank = kG == 2 ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;                 // issues the MMAs for the pair
  // Tile order: M-fastest (CTAs running together share a B tile) or N-fastest (they share an A
  // tile, so a large A is fetched from HBM once); see the host-side choice.
  auto tile_m = [&](int t) { return p.n_fastest ? t / p.n_tiles : t % p.m_tiles; };
  auto tile_n = [&](int t) { return p.n_fastest ? t % p.n_tiles : t / p.m_tiles; };
  const int first_tile = static_cast<int>(blockIdx.x) / kG;
  const int tile_step = static_cast<int>(gridDim.x) / kG;
  const int row_off = static_cast<int>(cta_rank) * kTileM;
  const int col_off = static_cast<int>(cta_rank) * (p.block_n / kG);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), kG * kEpiWarps);   // one arrival per epilogue warp
    }
    mbar_init(smem_u32(&ctrl->b_full), 1);
    ctrl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    if (p.tma_store) tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    if (kG == 2) {
      tmem_alloc_2cta(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(2 * p.acc_cols));
      tmem_relinquish_2cta();
    } else {
      tmem_alloc_1cta(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(2 * p.acc_cols));
      tmem_relinquish_1cta();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kG == 2) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  HY3D_TRACE_DECL(tr);
  // Set-up done: let the next kernel in the stream begin its own, then wait until the
  // previous one (which produced A and the scales) has completed.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer (all lanes walk the loop, lane 0 issues) ----------------
    {
      const bool issuer = lane == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (b_res && first_tile < total_units && issuer) {
        const uint32_t bf = smem_u32(&ctrl->b_full);
        const int n0 = tile_n(first_tile) * p.block_n;
        mbar_arrive_expect_tx(bf, b_res_bytes);
        for (int kb = 0; kb < p.num_kb; ++kb)
          tma_load_2d(b_res_base + kb * b_bytes, &tm_b, bf, kb * kBlockKBytes, n0);
      }
      __syncwarp();
      for (int unit = first_tile; ok && unit < total_units; unit += tile_step) {
        const int split = p.splits > 1 ? unit / total_tiles : 0;
        const int tile = unit - split * total_tiles;
        const int kb0 = split * p.kb_per_split;
        const int nkb = p.splits > 1 ? min(p.kb_per_split, p.num_kb - kb0) : p.num_kb;
        const int m0 = tile_m(tile) * (kTileM * kG) + row_off;
        const int n0 = tile_n(tile) * p.block_n + col_off;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, kDevTimeoutEmpty);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = smem_base + stage * stage_bytes;
          if (b_res) {
            HY3D_TRACE_FINE(3, tr, 20, kb);
#if defined(HY3D_TRACE) || defined(HY3D_KO)
            if (p.debug & 1) { if (issuer) mbar_arrive(full); } else
#endif
            if (issuer) {
              mbar_arrive_expect_tx(full, a_bytes);
              tma_load_2d(sa, &tm_a, full, kb * kBlockKBytes, m0);
            }
            HY3D_TRACE_FINE(3, tr, 21, kb);
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
            continue;
          }
#if defined(HY3D_TRACE) || defined(HY3D_KO)
          if (p.debug & 1) {
            if (leader && issuer) mbar_arrive(full);
          } else
#endif
          if (!issuer) {
            // only lane 0 issues
          } else if (kG == 1) {
            mbar_arrive_expect_tx(full, stage_bytes);
#pragma unroll
            for (int a = 0; a < kAtoms; ++a) {
              const int kx = ((kb0 + kb) * kAtoms + a) * kBlockKBytes;   // past K: zero-filled
              tma_load_2d(sa + a * a_bytes, &tm_a, full, kx, m0);
              tma_load_2d(sa + kAtoms * a_bytes + a * b_bytes, &tm_b, full, kx, n0);
            }
          } else {
            // Both CTAs credit their bytes to the leader's barrier; only the leader arrives.
            const uint32_t full_leader = map_to_cta(full, 0);
            if (leader) mbar_arrive_expect_tx(full, 2 * stage_bytes);
#pragma unroll
            for (int a = 0; a < kAtoms; ++a) {
              const int kx = ((kb0 + kb) * kAtoms + a) * kBlockKBytes;
              tma_load_2d_pair(sa + a * a_bytes, &tm_a, full_leader, kx, m0);
              tma_load_2d_pair(sa + kAtoms * a_bytes + a * b_bytes, &tm_b, full_leader, kx, n0);
            }
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread of the pair's leader CTA) ----------------
    // The tensor pipe accepts an MMA only when it can start it, so every cycle this thread
    // spends between two issues is a cycle the pipe idles: the loop is kept to one barrier
    // probe, four issues and one commit per stage.
    if (leader) {
      const bool issuer = lane == 0;
      const uint32_t idesc = make_idesc_i8(kTileM * kG, static_cast<uint32_t>(p.block_n), false);
      // Descriptor = (low word: address field + leading-dimension offset, high word: stride,
      // version, swizzle).  Only the 14-bit address field changes from stage to stage and from
      // K step to K step (+2 per 32 bytes), and it never carries out of its field, so the loop
      // keeps one running low word per operand.
      const uint64_t desc_const = make_smem_desc(0, 1024, 128);
      const uint32_t desc_hi = static_cast<uint32_t>(desc_const >> 32);
      const uint32_t lo_const = static_cast<uint32_t>(desc_const);
      const uint32_t a_lo0 = lo_const | ((smem_base & 0x3FFFFu) >> 4);
      const uint32_t stage_step = stage_bytes >> 4;
      const uint32_t a_atom = a_bytes >> 4, b_atom = b_bytes >> 4;
      const uint32_t b_off = static_cast<uint32_t>(kAtoms) * a_atom;
#if defined(HY3D_TRACE) || defined(HY3D_KO)
      const bool do_mma = !(p.debug & 4);
#else
      constexpr bool do_mma = true;
#endif
      int stage = 0;
      uint32_t phase = 0;
      uint32_t a_lo = a_lo0;
      bool ok = true;
      int it = 0;
      auto next_stage = [&]() {
        a_lo += stage_step;
        if (++stage == p.stages) { stage = 0; phase ^= 1; a_lo = a_lo0; }
      };
      auto wait_full = [&]() {
        const uint32_t bar = smem_u32(&ctrl->full[stage]);
        bool r = mbar_test_wait(bar, phase);
        if (__all_sync(0xffffffffu, r)) return true;
        if (!r) r = mbar_wait<true>(bar, phase, abort_flag, kDevTimeoutFull);
        return __all_sync(0xffffffffu, r) != 0;
      };
      auto commit_empty = [&]() {
        // Frees the stage (in both CTAs of a pair) once these MMAs have read it.
        if (kG == 1) tc_commit_1cta(smem_u32(&ctrl->empty[stage]));
        else tc_commit_2cta(smem_u32(&ctrl->empty[stage]), 3);
      };
      const uint32_t b_res_lo0 = lo_const | ((b_res_base & 0x3FFFFu) >> 4);
      if (b_res && first_tile < total_units) {
        ok = mbar_wait(smem_u32(&ctrl->b_full), 0, abort_flag, kDevTimeoutFull);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after_sync();
      }
      for (int unit = first_tile; ok && unit < total_units; unit += tile_step, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        // K range of this unit; only the last range of a matrix can end in a ragged stage
        const int kb0 = p.splits > 1 ? (unit / total_tiles) * p.kb_per_split : 0;
        const int nkb = p.splits > 1 ? min(p.kb_per_split, p.num_kb - kb0) : p.num_kb;
        const int full_kb = (kb0 + nkb == p.num_kb && p.last_ksteps != 4 * kAtoms) ? nkb - 1 : nkb;
        ok = mbar_wait(smem_u32(&ctrl->tmem_empty[buf]), acc_phase ^ 1, abort_flag,
                       kDevTimeoutTmemEmpty);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (issuer) HY3D_TRACE_EVENT(1, tr, 6, it);
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.acc_cols);
        uint32_t acc = 0;   // the first MMA of a tile overwrites the accumulator
        if (b_res) {
          // A from the ring, B from its resident block of the same K index.
          uint32_t xb = b_res_lo0;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            ok = wait_full();
            if (!ok) break;
            if (issuer) HY3D_TRACE_FINE(1, tr, 22, kb);
            const int ksteps = kb + 1 < p.num_kb ? 4 : p.last_ksteps;
            if (issuer) {
              if (do_mma) {
                for (int k = 0; k < ksteps; ++k)
                  mma_i8_lohi<kG>(d_tmem, a_lo + 2 * k, xb + 2 * k, desc_hi, idesc, k ? 1u : acc);
              }
              commit_empty();
              HY3D_TRACE_FINE(1, tr, 23, kb);
            }
            acc = 1u;
            next_stage();
            xb += b_atom;
          }
          if (ok && issuer) {
            HY3D_TRACE_EVENT(1, tr, 3, it);
            tc_commit_1cta(smem_u32(&ctrl->tmem_full[buf]));
          }
          __syncwarp();
          continue;
        }
        for (int kb = 0; kb < full_kb; ++kb) {
          ok = wait_full();
          if (!ok) break;
          if (issuer) {
            if (do_mma) {
              uint32_t xa = a_lo, xb = a_lo + b_off;
#pragma unroll
              for (int a = 0; a < kAtoms; ++a) {
                mma_i8_lohi<kG>(d_tmem, xa, xb, desc_hi, idesc, a ? 1u : acc);
                mma_i8_lohi<kG>(d_tmem, xa + 2, xb + 2, desc_hi, idesc, 1u);
                mma_i8_lohi<kG>(d_tmem, xa + 4, xb + 4, desc_hi, idesc, 1u);
                mma_i8_lohi<kG>(d_tmem, xa + 6, xb + 6, desc_hi, idesc, 1u);
                xa += a_atom;
                xb += b_atom;
              }
            }
            commit_empty();
          }
          acc = 1u;
          next_stage();
        }
        if (ok && full_kb < nkb) {   // ragged last stage: fewer K steps
          ok = wait_full();
          if (ok) {
            if (issuer) {
              if (do_mma) {
                for (int k = 0; k < p.last_ksteps; ++k) {
                  const uint32_t at = static_cast<uint32_t>(k >> 2), kk = static_cast<uint32_t>(k & 3);
                  mma_i8_lohi<kG>(d_tmem, a_lo + at * a_atom + 2 * kk,
                                  a_lo + b_off + at * b_atom + 2 * kk, desc_hi, idesc, k ? 1u : acc);
                }
              }
              commit_empty();
            }
            acc = 1u;
            next_stage();
          }
        }
        if (ok && issuer) {
          HY3D_TRACE_EVENT(1, tr, 3, it);
          if (kG == 1) tc_commit_1cta(smem_u32(&ctrl->tmem_full[buf]));
          else tc_commit_2cta(smem_u32(&ctrl->tmem_full[buf]), 3);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;            // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;        // which of the warps sharing that quarter
    const int row_in_tile = quarter * 32 + lane;
    const int et = threadIdx.x - 64;         // 0..255
    const bool geglu = kEpi == HY3D_EPI_GEGLU;
    const bool gelu = kEpi == HY3D_EPI_GELU;
    const int64_t ldo = geglu ? (p.N >> 1) : p.N;
    const uint32_t stage_buf = staging_base + static_cast<uint32_t>((warp - 2) * p.store_bufs) * kSlabBytes;
    const int acc_per_slab = geglu ? 2 * kSlabCols : kSlabCols;
    // The accumulator buffer is handed back to the leader's MMA warp (its own CTA or the peer).
    // One arrival per warp: every lane's tcgen05.ld has completed (its own wait::ld), the
    // warp converges, then lane 0 signals.  (An arrival per thread would put 512 serialised
    // updates of one shared-memory word on the epilogue's critical path.)
    auto release_acc = [&](uint32_t bar) {
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (kG == 1 || leader) mbar_arrive(bar); else mbar_arrive_cluster(bar, 0);
      }
    };
    bool ok = true;
    int it = 0;
    int cur_n0 = -1;
    long long acc_tile = 0, acc_wait = 0;   // per-role cycle totals of a -DHY3D_TRACE build
    const bool scaled = p.out_dtype != HY3D_S32;
    // The activation scale of the NEXT tile's row is fetched one tile ahead, and the
    // per-column scales / bias are refilled only when the tile column changes (with the grid
    // a multiple of the column count, a CTA keeps its column for the whole launch).
    float as_next = 0.0f;
    // Tile coordinates advance by additions (tile += tile_step in the walk order), not by a
    // division per tile: (fast, slow) = (column, row unit) when N-fastest, else the reverse.
    const int fast_dim = p.n_fastest ? p.n_tiles : p.m_tiles;
    const int step_slow = tile_step / fast_dim, step_fast = tile_step - step_slow * fast_dim;
    int t_fast = 0, t_slow = 0;
    if (first_tile < total_tiles && p.splits == 1) {
      t_slow = first_tile / fast_dim;
      t_fast = first_tile - t_slow * fast_dim;
      const int m_first = (p.n_fastest ? t_slow : t_fast) * (kTileM * kG) + row_off + row_in_tile;
      if (scaled && m_first < p.M) as_next = p.act_scale[m_first];
    }
    for (int tile = first_tile; tile < total_units; tile += tile_step, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      int split = 0;
      if (p.splits > 1) {   // few tiles per CTA here: plain divisions
        split = tile / total_tiles;
        const int tl = tile - split * total_tiles;
        t_slow = p.n_fastest ? tile_m(tl) : tile_n(tl);
        t_fast = p.n_fastest ? tile_n(tl) : tile_m(tl);
      }
      const int m0 = (p.n_fastest ? t_slow : t_fast) * (kTileM * kG) + row_off;
      const int n0 = (p.n_fastest ? t_fast : t_slow) * p.block_n;
      float as = as_next;
      if (p.splits == 1) {
        t_fast += step_fast;
        t_slow += step_slow;
        if (t_fast >= fast_dim) { t_fast -= fast_dim; ++t_slow; }
        as_next = 0.0f;
        if (scaled && tile + tile_step < total_tiles) {
          const int mn = (p.n_fastest ? t_slow : t_fast) * (kTileM * kG) + row_off + row_in_tile;
          if (mn < p.M) as_next = p.act_scale[mn];
        }
      }
      if (scaled && n0 != cur_n0) {
        epi_bar_sync();            // every warp is done reading the previous columns
        for (int c = et; c < p.block_n; c += kEpiThreads) {
          const int n = n0 + c;
          ctrl->ws[c] = n < p.N ? load_scalar(p.w_scale, p.ws_dtype, n) : 0.0f;
          ctrl->bs[c] = (p.bias && n < p.N) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
        }
        epi_bar_sync();
        cur_n0 = n0;
      }
      const long long w0c = HY3D_CLK();
      if (ok) ok = mbar_wait(smem_u32(&ctrl->tmem_full[buf]), acc_phase, abort_flag,
                             kDevTimeoutTmemFull);
      const long long w1c = HY3D_CLK();
      acc_wait += w1c - w0c;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;   // warp-uniform; the named barriers above stay balanced
      tc_fence_after_sync();
      HY3D_EPI_TRACE(4, it);
      const int m = m0 + row_in_tile;
      const bool row_ok = m < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * p.acc_cols);
      const float* wsb = ctrl->ws;
      const float* bsb = ctrl->bs;
      bool arrived = false;
#if defined(HY3D_TRACE) || defined(HY3D_KO)
      const bool skip_epilogue = (p.debug & 2) != 0;
#else
      constexpr bool skip_epilogue = false;
#endif
      if (p.splits > 1 && p.tma_store && !skip_epilogue) {
        // Split-K partials: raw int32 accumulators through the same staging buffers and bulk
        // stores, a slab being 32 rows x 16 int32 columns (64 bytes per row).  Each K range has
        // its own M-padded matrix in the workspace, so rows past M land in padding.
        const int nslab16 = p.block_n >> 4;
        const int out_row = split * p.m_rows_pad + m0 + quarter * 32;
        const int pend = p.store_bufs - 1;
        int sb = 0;
        for (int s = half; s < nslab16; s += kWarpsPerQuarter) {
          uint32_t r16[16];
          __syncwarp();
          tmem_ld_x16(t_row + 16 * s, r16);
          tmem_ld_wait();
          if (s + kWarpsPerQuarter >= nslab16) {
            tc_fence_before_sync();
            release_acc(smem_u32(&ctrl->tmem_empty[buf]));
            arrived = true;
          }
          slab_store(r16, stage_buf + sb * kSlabBytes, lane, pend, &tm_o, (n0 + 16 * s) * 4, out_row,
                     n0 + 16 * s < p.N);
          if (++sb == p.store_bufs) sb = 0;
        }
      } else if (p.tma_store && !skip_epilogue) {
        const int nslab = p.block_n / acc_per_slab;
        const int out_row = m0 + quarter * 32;
        const bool rows_in = out_row < p.M;
        const int pend = p.store_bufs - 1;
        int sb = 0;
        if (kEpi != HY3D_EPI_GEGLU) {
          // Each warp takes every kWarpsPerQuarter-th slab of its quarter; once its last
          // tcgen05.ld has landed the accumulator buffer is handed back to the MMA warp.
          for (int s = half; s < nslab; s += kWarpsPerQuarter) {
            uint32_t r[32], packed[16];
            __syncwarp();
            tmem_ld_x32(t_row + s * kSlabCols, r);
            tmem_ld_wait();
            if (s + kWarpsPerQuarter >= nslab) {
              tc_fence_before_sync();
              release_acc(smem_u32(&ctrl->tmem_empty[buf]));
              arrived = true;
            }
            slab_math<kBf16, kEpi>(r, as, wsb + s * kSlabCols, bsb + s * kSlabCols, packed);
            slab_store(packed, stage_buf + sb * kSlabBytes, lane, pend, &tm_o,
                       (n0 + s * kSlabCols) * 2, out_row, rows_in && n0 + s * kSlabCols < p.N);
            if (++sb == p.store_bufs) sb = 0;
          }
        } else {
          for (int s = half; s < nslab; s += kWarpsPerQuarter) {
            const int c0 = s * acc_per_slab;
            uint32_t packed[16];
            __syncwarp();
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              uint32_t rv[16], rg[16];
              const int cb = c0 + 32 * b;
              tmem_ld_x16(t_row + cb, rv);
              tmem_ld_x16(t_row + cb + 16, rg);
              tmem_ld_wait();
              slab_math_geglu<kBf16>(rv, rg, as, wsb + cb, bsb + cb, packed + 8 * b);
            }
            slab_store(packed, stage_buf + sb * kSlabBytes, lane, pend, &tm_o, ((n0 + c0) >> 1) * 2,
                       out_row, rows_in && ((n0 + c0) >> 1) < ldo);
            if (++sb == p.store_bufs) sb = 0;
          }
        }
      } else if (p.tma_store) {
        // diagnostic run: epilogue work skipped
      } else if (!geglu) {
        for (int c = 16 * half; c < p.block_n; c += 16 * kWarpsPerQuarter) {
          uint32_t r[16];
          __syncwarp();
          tmem_ld_x16(t_row + c, r);
          tmem_ld_wait();
          const int n = n0 + c;
          if (!row_ok || n >= p.N) {
            // nothing to store for this row / column block
          } else if (p.out_dtype == HY3D_S32) {
            int4* dst = reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(p.out) + split * p.split_stride +
                                                static_cast<int64_t>(m) * ldo + n);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[j] = make_int4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
            float y[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              y[j] = fmaf(static_cast<float>(static_cast<int32_t>(r[j])), as * wsb[c + j], bsb[c + j]);
              if (gelu) y[j] = gelu_erf(y[j]);
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) +
                                                  static_cast<int64_t>(m) * ldo + n);
            dst[0] = make_uint4(pack2(y[0], y[1], p.out_dtype), pack2(y[2], y[3], p.out_dtype),
                                pack2(y[4], y[5], p.out_dtype), pack2(y[6], y[7], p.out_dtype));
            dst[1] = make_uint4(pack2(y[8], y[9], p.out_dtype), pack2(y[10], y[11], p.out_dtype),
                                pack2(y[12], y[13], p.out_dtype), pack2(y[14], y[15], p.out_dtype));
          }
        }
      } else {
        // Columns come in blocks of 32: 16 "value" columns then their 16 "gate" columns.
        for (int c = 32 * half; c < p.block_n; c += 32 * kWarpsPerQuarter) {
          uint32_t rv[16], rg[16];
          __syncwarp();
          tmem_ld_x16(t_row + c, rv);
          tmem_ld_x16(t_row + c + 16, rg);
          tmem_ld_wait();
          const int n = n0 + c;
          if (row_ok && n < p.N) {
            float y[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float v = fmaf(static_cast<float>(static_cast<int32_t>(rv[j])), as * wsb[c + j],
                                   bsb[c + j]);
              const float g = fmaf(static_cast<float>(static_cast<int32_t>(rg[j])),
                                   as * wsb[c + 16 + j], bsb[c + 16 + j]);
              y[j] = v * gelu_erf(g);
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) +
                                                  static_cast<int64_t>(m) * ldo + (n >> 1));
            dst[0] = make_uint4(pack2(y[0], y[1], p.out_dtype), pack2(y[2], y[3], p.out_dtype),
                                pack2(y[4], y[5], p.out_dtype), pack2(y[6], y[7], p.out_dtype));
            dst[1] = make_uint4(pack2(y[8], y[9], p.out_dtype), pack2(y[10], y[11], p.out_dtype),
                                pack2(y[12], y[13], p.out_dtype), pack2(y[14], y[15], p.out_dtype));
          }
        }
      }
      HY3D_EPI_TRACE(5, it);
      acc_tile += HY3D_CLK() - w1c;
      __syncwarp();
      if (!arrived) {
        tc_fence_before_sync();
        release_acc(smem_u32(&ctrl->tmem_empty[buf]));
      }
    }
    if (threadIdx.x == 64) {
      HY3D_TRACE_RAW(4, acc_tile); HY3D_TRACE_RAW(5, acc_wait); HY3D_TRACE_RAW(6, it);
    }
    // Global writes of the bulk stores must be complete before the CTA retires.
    if (p.tma_store && lane == 0) tma_store_wait_all<0>();
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Let copies that may still be in flight land before the shared memory is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  // Neither CTA of a pair may retire while the other can still touch its shared memory,
  // barriers or tensor memory.
  if (kG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (kG == 2) tmem_dealloc_2cta(tmem_base, static_cast<uint32_t>(2 * p.acc_cols));
    else tmem_dealloc_1cta(tmem_base, static_cast<uint32_t>(2 * p.acc_cols));
  }
}

// Eight consecutive per-column parameters (16-byte aligned start) as floats, one or two vector loads.
__device__ __forceinline__ void load8_as_float(const void* p, int dtype, int n, float (&f)[8]) {
  if (dtype == HY3D_F32) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + n));
    const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + n) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    return;
  }
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + n));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dtype == HY3D_BF16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

// Split-K tail: sums the int32 partials of every K range (exact) and applies the layer's
// epilogue with the formula and roundings of the GEMM kernel's own (acc * (as * ws) + b,
// optional exact-erf GELU, one rounding to the 16-bit type).  One thread per 8 output columns.
template <bool kBf16, int kEpi>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const int32_t* __restrict__ partial, int splits, int64_t split_stride,
                     const float* __restrict__ act_scale, const void* __restrict__ w_scale, int ws_dtype,
                     const void* __restrict__ bias, int bias_dtype, uint16_t* __restrict__ out,
                     int64_t M, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_cols = N >> 3;
  const int64_t total = M * vec_cols;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = idx / vec_cols;
    const int n = static_cast<int>(idx - m * vec_cols) << 3;
    int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int32_t* src = partial + m * N + n;
    int sidx = 0;
    for (; sidx + 4 <= splits; sidx += 4) {        // eight independent 16-byte loads in flight
      int4 lo[4], hi[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        lo[u] = __ldcs(reinterpret_cast<const int4*>(src + (sidx + u) * split_stride));
        hi[u] = __ldcs(reinterpret_cast<const int4*>(src + (sidx + u) * split_stride) + 1);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        acc[0] += lo[u].x; acc[1] += lo[u].y; acc[2] += lo[u].z; acc[3] += lo[u].w;
        acc[4] += hi[u].x; acc[5] += hi[u].y; acc[6] += hi[u].z; acc[7] += hi[u].w;
      }
    }
    for (; sidx < splits; ++sidx) {
      const int4 lo = __ldcs(reinterpret_cast<const int4*>(src + sidx * split_stride));
      const int4 hi = __ldcs(reinterpret_cast<const int4*>(src + sidx * split_stride) + 1);
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
    const float as = act_scale[m];
    float wsf[8], bf[8];
    load8_as_float(w_scale, ws_dtype, n, wsf);
    if (bias) {
      load8_as_float(bias, bias_dtype, n, bf);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) bf[j] = 0.0f;
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float y[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        y[u] = __fmaf_rn(static_cast<float>(acc[j + u]), __fmul_rn(as, wsf[j + u]), bf[j + u]);
        if (kEpi == HY3D_EPI_GELU) y[u] = gelu_erf(y[u]);
      }
      w[j >> 1] = pack2t<kBf16>(y[0], y[1]);
    }
    *reinterpret_cast<uint4*>(out + m * N + n) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace

// Split-K plan for a dense layer: how many K ranges pay (1 = none).  Splitting serves launches
// whose tiles leave most SMs idle while each tile walks a long K alone (the M = 257 image-encoder
// layers with K = 6144): the ranges run side by side and a second small kernel adds them up.
int dense_splitk_plan(int64_t M, int64_t N, int64_t K, int epilogue) {
  if (epilogue == HY3D_EPI_GEGLU || (N & 7) || M <= 0) return 1;
  const int sms = device_sm_count() > 0 ? device_sm_count() : 148;
  const int64_t bn = N <= 128 ? N : 256;
  const int64_t tiles = ((M + kTileM - 1) / kTileM) * ((N + bn - 1) / bn);
  const int64_t num_kb = (K + kBlockKBytes - 1) / kBlockKBytes;
  if (tiles * 2 > sms || num_kb < 16) return 1;
  // Measured cost model (microseconds): a tile walks its K blocks at ~0.27 us each; every range
  // writes and re-reads an M-padded int32 matrix at ~5 TB/s; two launches cost ~6 us of fixed
  // time against ~3.5 us for one.  The split has to win by a tenth to be taken.
  const double part_us = static_cast<double>((M + kTileM - 1) / kTileM * kTileM) * N * 4.0 * 2.0 / 5.0e6;
  const double single = num_kb * 0.27 + 3.5;
  double best = single * 0.9;
  int best_s = 1;
  for (int64_t sp = 2; sp <= 16 && sp * tiles <= sms && sp * 4 <= num_kb; ++sp) {
    const double t = ((num_kb + sp - 1) / sp) * 0.27 + sp * part_us + 6.0;
    if (t < best) { best = t; best_s = static_cast<int>(sp); }
  }
  return best_s;
}

int gemm_dense(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale,
               int ws_dtype, const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M,
               int64_t N, int64_t K, int epilogue, int cta_group, int block_n,
               cudaStream_t stream, int splits = 1, int32_t* workspace = nullptr) {
  if (out_dtype != HY3D_F16 && out_dtype != HY3D_BF16 && out_dtype != HY3D_S32) return HY3D_ERR_ARG;
  if (epilogue < HY3D_EPI_LINEAR || epilogue > HY3D_EPI_GEGLU) return HY3D_ERR_ARG;
  if (out_dtype == HY3D_S32 && epilogue != HY3D_EPI_LINEAR) return HY3D_ERR_ARG;
  if (ws_dtype < HY3D_F16 || ws_dtype > HY3D_F32) return HY3D_ERR_ARG;
  if (bias && (bias_dtype < HY3D_F16 || bias_dtype > HY3D_F32)) return HY3D_ERR_ARG;
  if (cta_group < 0 || cta_group > 2) return HY3D_ERR_ARG;
  if (M < 0 || N <= 0 || K <= 0 || (K & 15) || (N & 15)) return HY3D_ERR_SHAPE;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return HY3D_ERR_SHAPE;
  const bool geglu = epilogue == HY3D_EPI_GEGLU;
  if (geglu && (N & 31)) return HY3D_ERR_SHAPE;
  if (M == 0) return HY3D_OK;
  if (!A || !B || !out) return HY3D_ERR_ARG;
  if (splits < 1 || splits > 64) return HY3D_ERR_ARG;
  if (splits > 1) {
    // K ranges as int32 partials in the caller's workspace, then the reduce + epilogue kernel.
    if (!workspace || out_dtype == HY3D_S32 || epilogue == HY3D_EPI_GEGLU || (N & 7)) return HY3D_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) || !act_scale || !w_scale) return HY3D_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(w_scale) | reinterpret_cast<uintptr_t>(bias)) & 15) return HY3D_ERR_SHAPE;
  }
  if (out_dtype != HY3D_S32 && (!act_scale || !w_scale)) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return HY3D_ERR_SHAPE;

  if (block_n == 0) {
    if (N <= 128) {
      block_n = static_cast<int>(N);
    } else {
      // Tile width (a multiple of the TMA-store slab) that minimises rounds x time per tile,
      // where rounds = ceil(tiles / SMs) and a tile costs its width plus a fixed per-stage
      // overhead worth ~94 columns of MMA time (measured).  A last tile that sticks out of N
      // is zero-filled on load and clipped on store.
      const int sms = device_sm_count();
      const int64_t m_tiles = (M + kTileM - 1) / kTileM;
      const int step = geglu ? 64 : 32;
      int64_t best = -1;
      const int nsm = sms > 0 ? sms : 148;
      for (int bn = 256; bn >= 128; bn -= step) {
        const int64_t n_tiles = (N + bn - 1) / bn;
        const int64_t tiles = m_tiles * n_tiles;
        // The grid is rounded down to a multiple of the column count (see the launch below).
        const int64_t grid = n_tiles <= nsm / 4 ? nsm - nsm % n_tiles : nsm;
        const int64_t rounds = (tiles + grid - 1) / grid;
        const int64_t cost = rounds * (bn + 94);
        if (best < 0 || cost < best) { best = cost; block_n = bn; }
      }
    }
  }
  if (block_n < 16 || block_n > 256 || (block_n & 15) || (geglu && (block_n & 31)))
    return HY3D_ERR_SHAPE;

  // CTA pairs need an even split of the B tile into two multiples of 16 rows.
  int group = cta_group;
  if (group == 0) {
    // CTA pairs halve the B traffic into shared memory, which is what bounds the tensor pipe
    // on deep-K problems (measured: 8192^3 2768 vs 2332 TOPS); with K >= 2048 they pay off
    // as soon as most SM pairs have a tile, with K >= 1024 once the grid holds several rounds
    // of 256-row tile pairs; on shorter K the per-tile hand-offs of a pair cost more.
    const int sms = device_sm_count() > 0 ? device_sm_count() : 148;
    const int64_t pair_tiles = ((M + 2 * kTileM - 1) / (2 * kTileM)) * ((N + block_n - 1) / block_n);
    const int64_t min_pair_tiles = K >= 2048 ? (sms / 2) * 4 / 5 : 4 * (sms / 2);
    group = (K >= 1024 && (block_n & 31) == 0 && pair_tiles >= min_pair_tiles) ? 2 : 1;
#ifdef HY3D_TRACE
    if (const char* e = getenv("HY3D_CTA_GROUP")) group = atoi(e) == 2 ? 2 : 1;
#endif
  }
  if (group == 2 && (block_n & 31)) {
    if (cta_group == 2) return HY3D_ERR_SHAPE;
    group = 1;
  }

  DenseArgs p;
  p.act_scale = act_scale; p.w_scale = w_scale; p.bias = bias; p.out = out;
  p.ws_dtype = ws_dtype; p.bias_dtype = bias_dtype; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.block_n = block_n;
  int acc_cols = 32;
  while (acc_cols < block_n) acc_cols <<= 1;
  p.acc_cols = acc_cols;
  p.m_tiles = static_cast<int>((M + kTileM * group - 1) / (kTileM * group));
  p.n_tiles = static_cast<int>((N + block_n - 1) / block_n);
  // Deep stages (two 128-byte K blocks, eight MMAs per barrier round trip) for CTA pairs on
  // deep K: a pair's per-stage hand-off crosses the cluster, and halving the number of
  // hand-offs is what lets pairs profit from their smaller shared-memory traffic.
  const int atoms = (group == 2 && K >= 1024 && splits == 1) ? 2 : 1;
  p.atoms = atoms;
  const int stage_k = kBlockKBytes * atoms;
  p.num_kb = static_cast<int>((K + stage_k - 1) / stage_k);
  const int k_last = static_cast<int>(K - static_cast<int64_t>(p.num_kb - 1) * stage_k);
  p.last_ksteps = (k_last + 31) / 32;
  p.splits = 1; p.kb_per_split = p.num_kb; p.split_stride = 0;
  const int final_dtype = out_dtype, final_epilogue = epilogue;
  void* final_out = out;
  if (splits > 1) {
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;      // no empty range
    p.splits = splits;
    p.m_rows_pad = p.m_tiles * kTileM * group;
    p.split_stride = static_cast<int64_t>(p.m_rows_pad) * N;
    p.out = workspace; p.out_dtype = out_dtype = HY3D_S32; p.epilogue = epilogue = HY3D_EPI_LINEAR;
    p.act_scale = nullptr;
  }
  p.tma_store = (out_dtype != HY3D_S32 && block_n % (geglu ? 2 * kSlabCols : kSlabCols) == 0) ? 1 : 0;
  if (p.splits > 1) p.tma_store = 1;   // 64-byte slabs of int32 partials (block_n is a multiple of 16)

  // Grid and tile order.  Tiles are walked N-fastest: CTAs running together share an A tile (a
  // large activation matrix is then fetched from HBM once, while the small B stays
  // L2-resident), and with the grid rounded down to a multiple of the column count every CTA
  // keeps ONE tile column for the whole launch, so its per-column scales and bias are staged
  // once and the epilogue warps never meet at a CTA-wide barrier again (measured faster or
  // equal on every sweep shape).
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  const int total_tiles = p.m_tiles * p.n_tiles;
  const int total_units = total_tiles * p.splits;
  const int max_clusters = sms / group;
  int clusters = total_units < max_clusters ? total_units : max_clusters;
  bool column_fixed = p.n_tiles == 1;
  p.n_fastest = 0;
  if (p.n_tiles > 1) {
    p.n_fastest = 1;
    if (p.n_tiles <= clusters / 4) { clusters -= clusters % p.n_tiles; column_fixed = true; }
  }
#ifdef HY3D_TRACE
  if (const char* e = getenv("HY3D_ORDER")) {
    p.n_fastest = atoi(e) ? 1 : 0;
    clusters = total_tiles < max_clusters ? total_tiles : max_clusters;
    column_fixed = p.n_tiles == 1;
    if (p.n_fastest && p.n_tiles <= clusters / 4) { clusters -= clusters % p.n_tiles; column_fixed = true; }
  }
#endif

  // Shared memory: [pipeline stages][resident B tile][store staging][control block].
  // A single CTA's load rate from L2 (about 64 bytes per clock) is what paces short-K tiles:
  // 128 x block_n outputs need (128 + block_n) x K operand bytes per tile.  Where a CTA keeps
  // its tile column and the column's B tile fits beside at least four A stages, B is loaded
  // once and only A streams: 128 x K bytes per tile.
  const int a_stage = kTileM * kBlockKBytes;
  const int b_tile_bytes = p.num_kb * block_n * kBlockKBytes;
  const int ctrl_bytes = static_cast<int>(sizeof(DenseCtrl));
  const int staging1 = kEpiWarps * kSlabBytes;
  int b_resident = 0, store_bufs = 2, stages = 0, stage_bytes = 0;
  if (group == 1 && atoms == 1 && column_fixed && p.splits == 1 && total_tiles >= 2 * clusters) {
    // One staging buffer per epilogue warp: measured faster than two here (a warp that must
    // wait for its previous store to leave shared memory paces the store stream, and the
    // loads queue behind fewer stores).
    const int st = (kSmemLimit - ctrl_bytes - staging1 - b_tile_bytes) / a_stage;
    if (st >= 4) { b_resident = 1; store_bufs = 1; stages = st; stage_bytes = a_stage; }
  }
#if defined(HY3D_TRACE) || defined(HY3D_KO)
  if (const char* e = getenv("HY3D_B_RESIDENT")) { if (!atoi(e)) b_resident = 0; }
#endif
  if (!b_resident) {
    stage_bytes = atoms * (a_stage + (block_n / group) * kBlockKBytes);
    // Two staging buffers per epilogue warp unless that costs one of fewer than four pipeline stages.
    store_bufs = 2;
    const int fixed2 = ctrl_bytes + 2 * staging1, fixed1 = ctrl_bytes + staging1;
    const int stages2 = (kSmemLimit - fixed2) / stage_bytes, stages1 = (kSmemLimit - fixed1) / stage_bytes;
    if (stages2 < 4 && stages1 > stages2) store_bufs = 1;
#ifdef HY3D_TRACE
    if (const char* e = getenv("HY3D_STORE_BUFS")) store_bufs = atoi(e) == 1 ? 1 : 2;
#endif
    stages = (kSmemLimit - ctrl_bytes - store_bufs * staging1) / stage_bytes;
  }
  p.b_resident = b_resident;
  p.store_bufs = store_bufs;
  const int fixed = ctrl_bytes + store_bufs * staging1 + (b_resident ? b_tile_bytes : 0);
  if (stages > kMaxStages) stages = kMaxStages;
#ifdef HY3D_TRACE
  if (const char* e = getenv("HY3D_STAGES")) { const int v = atoi(e); if (v >= 2 && v < stages) stages = v; }
#endif
  if (stages < 2) return HY3D_ERR_SHAPE;
  p.stages = stages;
  p.debug = 0;
#if defined(HY3D_TRACE) || defined(HY3D_KO)
  { const char* e = getenv("HY3D_DEBUG"); p.debug = e ? atoi(e) : 0; }
#endif
  const int smem_bytes = stages * stage_bytes + fixed;

  CUtensorMap tm_a, tm_b, tm_o;
  int rc = encode_tmap_2d_u8(&tm_a, A, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                             static_cast<uint64_t>(K), kBlockKBytes, kTileM, 128);
  if (rc != HY3D_OK) return rc;
  rc = encode_tmap_2d_u8(&tm_b, B, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                         static_cast<uint64_t>(K), kBlockKBytes,
                         static_cast<uint32_t>(block_n / group), 128);
  if (rc != HY3D_OK) return rc;
  if (p.splits > 1) {
    const uint64_t row_bytes = static_cast<uint64_t>(N) * 4;
    rc = encode_tmap_2d_u8(&tm_o, workspace, row_bytes, static_cast<uint64_t>(p.splits) * p.m_rows_pad,
                           row_bytes, 64, 32, 64);
    if (rc != HY3D_OK) return rc;
  } else if (p.tma_store) {
    const uint64_t row_bytes = static_cast<uint64_t>(geglu ? N / 2 : N) * 2;
    rc = encode_tmap_2d_u8(&tm_o, out, row_bytes, static_cast<uint64_t>(M), row_bytes,
                           kSlabCols * 2, 32, 64);
    if (rc != HY3D_OK) return rc;
  } else {
    tm_o = tm_a;   // unused by the kernel
  }

  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const DenseArgs);
  // [0]: one CTA per tile, [1]: CTA pairs, [2]: CTA pairs with deep (two-block) stages.
#define HY3D_DENSE_ROW(G, A)                                                              \
  {{gemm_dense_kernel<false, HY3D_EPI_LINEAR, G, A>, gemm_dense_kernel<false, HY3D_EPI_GELU, G, A>, \
    gemm_dense_kernel<false, HY3D_EPI_GEGLU, G, A>},                                        \
   {gemm_dense_kernel<true, HY3D_EPI_LINEAR, G, A>, gemm_dense_kernel<true, HY3D_EPI_GELU, G, A>,   \
    gemm_dense_kernel<true, HY3D_EPI_GEGLU, G, A>}}
  static const KernelFn kernels[3][2][3] = {HY3D_DENSE_ROW(1, 1), HY3D_DENSE_ROW(2, 1), HY3D_DENSE_ROW(2, 2)};
#undef HY3D_DENSE_ROW
  // Raw int32 output runs the direct-store path of the <false, LINEAR> instance.
  const int ki = out_dtype == HY3D_BF16 ? 1 : 0;
  const int variant = (group == 2 && atoms == 2) ? 2 : group - 1;
  const KernelFn kernel = kernels[variant][ki][epilogue];
  rc = ensure_max_smem(reinterpret_cast<const void*>(kernel), kSmemLimit);
  if (rc != HY3D_OK) return rc;
  const int grid = group * clusters;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[1] = pdl_attribute();
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(group);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_o, p) != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  if (p.splits > 1) {
    const int64_t vecs = M * (N >> 3);
    int64_t blocks = (vecs + 255) / 256;
    if (blocks > sms * 8) blocks = sms * 8;
    cudaLaunchConfig_t rcfg = {};
    rcfg.gridDim = dim3(static_cast<unsigned>(blocks));
    rcfg.blockDim = dim3(256);
    rcfg.stream = stream;
    cudaLaunchAttribute rattr[1];
    rattr[0] = pdl_attribute();
    rcfg.attrs = rattr;
    rcfg.numAttrs = 1;
    const int32_t* part = workspace;
    uint16_t* o16 = static_cast<uint16_t*>(final_out);
    const int Ni = static_cast<int>(N);
    cudaError_t err;
#define HY3D_SPLITK_REDUCE(BF, EP)                                                                    \
  err = cudaLaunchKernelEx(&rcfg, splitk_reduce_kernel<BF, EP>, part, p.splits, p.split_stride, act_scale, \
                           w_scale, ws_dtype, bias, bias_dtype, o16, M, Ni)
    if (final_dtype == HY3D_BF16) {
      if (final_epilogue == HY3D_EPI_GELU) HY3D_SPLITK_REDUCE(true, HY3D_EPI_GELU);
      else HY3D_SPLITK_REDUCE(true, HY3D_EPI_LINEAR);
    } else {
      if (final_epilogue == HY3D_EPI_GELU) HY3D_SPLITK_REDUCE(false, HY3D_EPI_GELU);
      else HY3D_SPLITK_REDUCE(false, HY3D_EPI_LINEAR);
    }
#undef HY3D_SPLITK_REDUCE
    if (err != cudaSuccess) { cudaGetLastError(); return HY3D_ERR_CUDA; }
  }
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace dense

using dense::gemm_dense;
using dense::dense_splitk_plan;

}  // namespace hy3d
