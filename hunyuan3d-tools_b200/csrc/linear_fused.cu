// Whole dense W8A8 linear layer as ONE kernel for sm_100a, with the quantised activations
// resident in shared memory:
//     out(M,N) = epilogue( quantise_rows(x(M,K)) * B(N,K)^T )
//
// A CTA owns a block of 128 tokens at a time.  Dedicated quantiser warps read the block's
// fp16 / bf16 rows once with 16-byte loads, reduce each row's absmax with shuffles and write
// the int8 codes STRAIGHT into the 128-byte-swizzled shared-memory operand tiles for the whole
// K (ceil(K/128) tiles of 128 rows x 128 B), so the int8 activations never exist in global
// memory.  The MMA thread then runs every weight tile assigned to the CTA against that
// resident block (tile columns innermost); only the weights stream through a TMA ring.  The
// per-token scales stay in shared memory for the epilogue.  With K <= 640 two operand blocks
// fit, so the quantiser prepares block j+1 under the MMAs of block j; longer rows (K <= 1280)
// use one block, and the rows of the CTA's next block are pulled into L2 ahead of time with a
// bulk prefetch so the serial quantise phase reads from L2, not from HBM.
//
// Roles by warp (832 threads):
//   warp 0        TMA producer of the weight tiles (block_n rows x 128 B, 128-byte swizzle)
//   warp 1        tensor-memory owner; one thread issues tcgen05.mma kind::i8
//   warps 2-9     epilogue, two warps per 32-lane quarter of tensor memory: tcgen05.ld,
//                 acc * (act_scale[m] * w_scale[n]) + bias[n] (+ GELU / GEGLU), TMA store
//   warps 10-25   quantiser (8 rows of the block each)
// Work is the list of (token block, weight tile) units in token-block-major order; every CTA
// takes one contiguous range of it, so a block is quantised once per CTA that touches it.
//
// The arithmetic is that of quantize_rows_kernel and gemm_dense_kernel (same helper
// functions), so the output is bit-identical to the two-launch path.
#include "common.cuh"

namespace hy3d {
int ensure_max_smem(const void* kernel, int bytes);

namespace fused {
namespace {

constexpr int kTileM = 128;
constexpr int kAtomBytes = kTileM * 128;     // one 128-deep K slice of the token block
constexpr int kMaxAtoms = 10;                // K <= 1280
constexpr int kMaxStages = 8;
// 24 worker warps split between the two ALU-heavy roles (template parameter kEW = epilogue
// warps, a multiple of 4 so that every 32-lane quarter of tensor memory gets the same number):
// 16 + 8 when a token block feeds many output columns, 8 + 16 when the rows are long.
constexpr int kWorkerWarps = 24;
constexpr int kMaxEpiWarps = 16;
constexpr int kThreads = 64 + 32 * kWorkerWarps;
constexpr int kSlabCols = 32;                // output columns per TMA store
constexpr int kSlabBytes = 32 * kSlabCols * 2;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxVecs = 5;                  // 16-byte vectors a quantiser lane holds per row
constexpr int kScaleSlots = 4;               // per-token scale buffers, indexed by block & 3

struct FusedArgs {
  const uint16_t* x;      // fp16 / bf16 activations (M, K), row pitch ldx elements
  int64_t ldx;
  float* scale_out;       // optional: per-token scales (M) written to global memory
  const void* w_scale;
  const void* bias;
  int ws_dtype, bias_dtype;
  int M, N, K;
  int block_n, stages, acc_cols, store_bufs;
  int m_blocks, n_tiles, atoms, last_ksteps;
  int a_bufs;             // resident token blocks (1 or 2)
  int unit_align;         // CTA ranges start at multiples of this many units
  int q_lanes_log2;       // quantiser lanes per row = 1 << q_lanes_log2 (2..5)
  int q_vecs;             // 16-byte vectors per lane and row (<= kMaxVecs)
  int debug;              // knock-out switches of -DHY3D_TRACE builds (always 0 in the shipped library)
};

struct __align__(16) FusedCtrl {
  float as[kScaleSlots][kTileM];   // per-token scales of the resident blocks
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t a_full[2];
  uint64_t a_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// First and one-past-last unit of a CTA: contiguous, balanced to within unit_align units.
__device__ __forceinline__ void unit_range(const FusedArgs& p, int& lo, int& hi) {
  const long long total = static_cast<long long>(p.m_blocks) * p.n_tiles;
  const long long chunks = (total + p.unit_align - 1) / p.unit_align;
  const long long c = blockIdx.x, g = gridDim.x;
  long long a = (c * chunks / g) * p.unit_align, b = ((c + 1) * chunks / g) * p.unit_align;
  lo = static_cast<int>(a < total ? a : total);
  hi = static_cast<int>(b < total ? b : total);
}

__device__ __forceinline__ void prefetch_l2_bulk(const void* ptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
}

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

// 16 accumulator columns of one row -> 16 outputs (rescale, bias, optional GELU, pack) written
// as two 16-byte pieces into the row's 64-byte line of the staging buffer (64-byte swizzle:
// 16-byte chunk c of row r sits at c ^ ((r >> 1) & 3)); `hi` selects the line's second half.
template <bool kBf16, int kEpi>
__device__ __forceinline__ void chunk_math_store(const uint32_t (&r)[16], float as, const float* wsb,
                                                 const float* bsb, uint32_t buf_addr, int lane, int hi) {
  const float2 as2 = make_float2(as, as);
  uint32_t packed[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 w4 = *reinterpret_cast<const float4*>(wsb + 4 * q);
    const float4 b4 = *reinterpret_cast<const float4*>(bsb + 4 * q);
    const float2 s01 = __fmul2_rn(as2, make_float2(w4.x, w4.y));
    const float2 s23 = __fmul2_rn(as2, make_float2(w4.z, w4.w));
    const float2 a01 = make_float2(static_cast<float>(static_cast<int32_t>(r[4 * q + 0])),
                                   static_cast<float>(static_cast<int32_t>(r[4 * q + 1])));
    const float2 a23 = make_float2(static_cast<float>(static_cast<int32_t>(r[4 * q + 2])),
                                   static_cast<float>(static_cast<int32_t>(r[4 * q + 3])));
    float2 y01 = __ffma2_rn(a01, s01, make_float2(b4.x, b4.y));
    float2 y23 = __ffma2_rn(a23, s23, make_float2(b4.z, b4.w));
    if (kEpi == HY3D_EPI_GELU) {
      y01.x = gelu_erf(y01.x); y01.y = gelu_erf(y01.y); y23.x = gelu_erf(y23.x); y23.y = gelu_erf(y23.y);
    }
    packed[2 * q] = dense::pack2t<kBf16>(y01.x, y01.y);
    packed[2 * q + 1] = dense::pack2t<kBf16>(y23.x, y23.y);
  }
  const uint32_t row_addr = buf_addr + static_cast<uint32_t>(lane) * 64u;
  const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
  const uint32_t c0 = static_cast<uint32_t>(hi) * 2u;
  dense::st_shared_v4(row_addr + (((c0) ^ sw) << 4), packed[0], packed[1], packed[2], packed[3]);
  dense::st_shared_v4(row_addr + (((c0 + 1u) ^ sw) << 4), packed[4], packed[5], packed[6], packed[7]);
}

struct QuantCtx {
  uint32_t smem_base, a_block_bytes;
  int unit_lo, unit_hi, qw, lane;
  volatile int* abort_flag;
};

// The quantiser role of one warp: its rows of every token block in the CTA's range, a batch
// of 32 / G rows at a time (G lanes share a row, each holding kMaxVecs 16-byte vectors), with
// the loads of the next batch in flight while the current one is reduced, quantised and stored
// into the swizzled operand tiles.  kLg > 0 fixes G = 1 << kLg with exactly kMaxVecs vectors
// per lane at compile time (no predicates, store addresses = one base per batch + constants);
// kLg == 0 reads the geometry from the arguments.
template <bool kBf16, int kLg, int kRowsPerQuantWarp>
__device__ __forceinline__ void quantiser_role(const FusedArgs& p, FusedCtrl* ctrl, const QuantCtx& q) {
  const int lane = q.lane, qw = q.qw;
  const int lg = kLg > 0 ? kLg : p.q_lanes_log2;
  const int G = 1 << lg;
  const int sub = lane & (G - 1);
  const int rsub = lane >> lg;
  const int rpb_log2 = 5 - lg;                    // rows per batch = 32 / G
  constexpr int kRowsLog2 = kRowsPerQuantWarp == 16 ? 4 : 3;
  static_assert(kRowsPerQuantWarp == (1 << kRowsLog2), "8 or 16 rows per quantiser warp");
  const int bat_log2 = kRowsLog2 - rpb_log2;      // batches per block = rows per warp / rows per batch
  const int batches = 1 << bat_log2;
  const int nvec = p.K >> 3;
  const int V = kLg > 0 ? kMaxVecs : p.q_vecs;
  const int m_first = q.unit_lo / p.n_tiles;
  const int m_last = q.unit_hi > q.unit_lo ? (q.unit_hi - 1) / p.n_tiles : m_first - 1;
  const int total_batches = (m_last - m_first + 1) << bat_log2;
  const int row_in_warp0 = qw * kRowsPerQuantWarp + rsub;   // + t * rows_per_batch
  const uint16_t* lane_src = p.x + static_cast<int64_t>(sub) * 8;
  HY3D_TRACE_DECL(tr);

  // Pulls this warp's rows of token block m towards L2 (one bulk prefetch per row).
  auto prefetch_block = [&](int m) {
    if (m <= m_last && lane < kRowsPerQuantWarp) {
      const int64_t row = static_cast<int64_t>(m) * kTileM + qw * kRowsPerQuantWarp + lane;
      if (row < p.M) prefetch_l2_bulk(p.x + row * p.ldx, static_cast<uint32_t>(p.K) * 2u);
    }
  };
  auto load_batch = [&](int idx, uint4 (&v)[kMaxVecs]) {
    const int m = m_first + (idx >> bat_log2), t = idx & (batches - 1);
    const int64_t row = static_cast<int64_t>(m) * kTileM + row_in_warp0 + (t << rpb_log2);
    const bool row_ok = row < p.M;
    const uint4* src = reinterpret_cast<const uint4*>(lane_src + (row_ok ? row : 0) * p.ldx);
#pragma unroll
    for (int i = 0; i < kMaxVecs; ++i) {
#ifdef HY3D_TRACE
      if (p.debug & 4) { v[i] = make_uint4(0x3f803f80u, 0x40004000u, 0xbf80bf80u, 0x3f003f00u); continue; }
#endif
      if (kLg > 0) v[i] = row_ok ? __ldcs(src + i * G) : make_uint4(0, 0, 0, 0);
      else v[i] = (i < V && row_ok && sub + i * G < nvec) ? __ldcs(src + i * G) : make_uint4(0, 0, 0, 0);
    }
  };
  // Quantises one batch of rows held in registers into the resident block; false on abort.
  auto process_batch = [&](int idx, const uint4 (&v)[kMaxVecs]) -> bool {
    const int blk = idx >> bat_log2, t = idx & (batches - 1);
    const int m = m_first + blk;
    const int abuf = blk % p.a_bufs;
    const int row_local = row_in_warp0 + (t << rpb_log2);
    const int64_t row = static_cast<int64_t>(m) * kTileM + row_local;
    const bool row_ok = row < p.M;
    if (qw == 0 && lane == 0) HY3D_TRACE_FINE(0, tr, 7, idx);
    uint32_t amax2 = 0;
#pragma unroll
    for (int i = 0; i < kMaxVecs; ++i) quant::absmax8<kBf16>(v[i], amax2);
    float amax = quant::absmax_to_float<kBf16>(amax2);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      if (off < G) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    const float inv = __frcp_rn(scale);
    if (qw == 0 && lane == 0) HY3D_TRACE_FINE(0, tr, 8, idx);
    if (t == 0) {
      // The block's shared-memory tiles are free once the MMAs of the block that used them
      // before have completed.
      if (qw == 0 && lane == 0) HY3D_TRACE_EVENT(0, tr, 5, blk);
      if (!mbar_wait(smem_u32(&ctrl->a_empty[abuf]), (static_cast<uint32_t>(blk / p.a_bufs) & 1u) ^ 1u,
                     q.abort_flag, kDevTimeoutEmpty))
        return false;
    }
    if (sub == 0) {
      ctrl->as[blk & (kScaleSlots - 1)][row_local] = row_ok ? scale : 0.0f;
      if (p.scale_out && row_ok) p.scale_out[row] = scale;
    }
    const uint32_t row_base = q.smem_base + static_cast<uint32_t>(abuf) * q.a_block_bytes +
                              static_cast<uint32_t>(row_local) * 128u;
    const uint32_t sw = static_cast<uint32_t>(row_local) & 7u;
    const uint32_t sub8 = static_cast<uint32_t>(sub) << 3;
#pragma unroll
    for (int i = 0; i < kMaxVecs; ++i) {
      if (kLg > 0 || (i < V && sub + i * G < nvec)) {
        float f[8];
        quant::unpack8<kBf16>(v[i], f);
        const uint2 c8 = quant::quant8(f, scale, inv);   // rows past M hold zeros: codes 0
        // byte offset of these 8 codes in the row: sub8 + 8 * G * i; with G fixed the second
        // term is a constant, so the swizzled address is a per-batch base plus an immediate
        const uint32_t kc = static_cast<uint32_t>(i * G) << 3;
        const uint32_t kin = sub8 + (kc & 127u);          // < 256
        const uint32_t addr = row_base + ((kc >> 7) + (kin >> 7)) * kAtomBytes +
                              ((((kin & 127u) >> 4) ^ sw) << 4) + (kin & 8u);
        st_shared_v2(addr, c8.x, c8.y);
      }
    }
    if (qw == 0 && lane == 0) HY3D_TRACE_FINE(0, tr, 9, idx);
    if (t == batches - 1) {
      // The tensor core reads these tiles through the async proxy.
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->a_full[abuf]));
      if (qw == 0 && lane == 0) HY3D_TRACE_EVENT(0, tr, 6, blk);
      // Every load of this block has been issued.  The first block this warp cannot start
      // right away (its tiles are still being read by the MMAs) is pulled towards L2 now, so
      // that HBM keeps streaming while the quantiser waits and the rows are close when the
      // tiles come free.  Earlier prefetches would only queue ahead of the demand loads.
#ifdef HY3D_TRACE
      if (!(p.debug & 8))
#endif
      prefetch_block(m + p.a_bufs);
    }
    return true;
  };

  // Software pipeline over (block, batch): the loads of batch i+1 are in flight while batch i
  // is reduced, quantised and stored.
  uint4 va[kMaxVecs], vb[kMaxVecs];
  bool ok = true;
  if (total_batches > 0) load_batch(0, va);
  for (int i = 0; ok && i < total_batches; i += 2) {
    if (i + 1 < total_batches) load_batch(i + 1, vb);
    ok = process_batch(i, va);
    if (!ok || i + 1 >= total_batches) break;
    if (i + 2 < total_batches) load_batch(i + 2, va);
    ok = process_batch(i + 1, vb);
  }
}

template <bool kBf16, int kEpi, int kEW>
__global__ void __launch_bounds__(kThreads, 1)
linear_fused_kernel(const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_o,
                    const FusedArgs p) {
  constexpr int kEpiWarps = kEW;
  constexpr int kEpiPerQuarter = kEW / 4;
  constexpr int kQuantWarps = kWorkerWarps - kEW;
  constexpr int kRowsPerQuantWarp = kTileM / kQuantWarps;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t smem_base = smem_u32(smem_raw);
  if (smem_base & 1023u) {   // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(&g_device_status, 0, static_cast<int>(kDevBadAlignment));
    return;
  }
  const uint32_t a_block_bytes = static_cast<uint32_t>(p.atoms) * kAtomBytes;
  const uint32_t b_bytes = static_cast<uint32_t>(p.block_n) * 128u;
  const uint32_t b_base = smem_base + static_cast<uint32_t>(p.a_bufs) * a_block_bytes;
  const uint32_t staging_base = b_base + static_cast<uint32_t>(p.stages) * b_bytes;
  const size_t staging_off = static_cast<size_t>(p.a_bufs) * a_block_bytes +
                             static_cast<size_t>(p.stages) * b_bytes;
  float* wsb_all = reinterpret_cast<float*>(smem + staging_off +
                                            static_cast<size_t>(kEpiWarps) * p.store_bufs * kSlabBytes);
  FusedCtrl* ctrl = reinterpret_cast<FusedCtrl*>(reinterpret_cast<uint8_t*>(wsb_all) +
                                                 kMaxEpiWarps * 256 * sizeof(float));
  volatile int* abort_flag = &ctrl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int unit_lo, unit_hi;
  unit_range(p, unit_lo, unit_hi);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), kEpiWarps);   // one arrival per epilogue warp
      mbar_init(smem_u32(&ctrl->a_full[b]), kQuantWarps);     // one arrival per quantiser warp
      mbar_init(smem_u32(&ctrl->a_empty[b]), 1);
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    tmem_alloc_1cta(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(2 * p.acc_cols));
    tmem_relinquish_1cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  // Set-up done: let the next kernel in the stream begin its own, then wait until the
  // previous one (which produced x) has completed.
  pdl_launch_dependents();
  pdl_wait();
  HY3D_TRACE_DECL(tr);

  if (warp == 0) {
    // ---------------- TMA producer of the weight tiles (one thread) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = unit_lo; ok && u < unit_hi; ++u) {
        const int n0 = (u % p.n_tiles) * p.block_n;
        for (int a = 0; a < p.atoms; ++a) {
          ok = mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, kDevTimeoutEmpty);
          if (!ok) break;
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          mbar_arrive_expect_tx(full, b_bytes);
          // Columns past K and rows past N are zero-filled by the tensor map.
          tma_load_2d(b_base + static_cast<uint32_t>(stage) * b_bytes, &tm_b, full, a * 128, n0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread) ----------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_i8(kTileM, static_cast<uint32_t>(p.block_n), false);
      const uint64_t desc_const = make_smem_desc(0, 1024, 128);
      const uint32_t desc_hi = static_cast<uint32_t>(desc_const >> 32);
      const uint32_t lo_const = static_cast<uint32_t>(desc_const);
      const uint32_t a_lo0 = lo_const | ((smem_base & 0x3FFFFu) >> 4);
      const uint32_t b_lo0 = lo_const | ((b_base & 0x3FFFFu) >> 4);
      const uint32_t b_step = b_bytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t b_lo = b_lo0;
      bool ok = true;
      int it = 0, blk = -1, prev_m = -1, abuf = 0;
      for (int u = unit_lo; ok && u < unit_hi; ++u, ++it) {
        const int m = u / p.n_tiles;
        if (m != prev_m) {
          prev_m = m;
          ++blk;
          abuf = blk % p.a_bufs;
          // a long wait (a whole block is being quantised): park instead of polling
          ok = mbar_wait(smem_u32(&ctrl->a_full[abuf]), static_cast<uint32_t>(blk / p.a_bufs) & 1u,
                         abort_flag, kDevTimeoutQuant);
          if (!ok) break;
        }
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait(smem_u32(&ctrl->tmem_empty[buf]), acc_phase ^ 1, abort_flag,
                       kDevTimeoutTmemEmpty);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.acc_cols);
        HY3D_TRACE_EVENT(1, tr, 1, u - unit_lo);
        uint32_t a_lo = a_lo0 + static_cast<uint32_t>(abuf) * (a_block_bytes >> 4);
        uint32_t acc = 0;   // the first MMA of a unit overwrites the accumulator
        for (int a = 0; a < p.atoms; ++a) {
          const uint32_t bar = smem_u32(&ctrl->full[stage]);
          if (!mbar_test_wait(bar, phase)) {
            ok = mbar_wait<true>(bar, phase, abort_flag, kDevTimeoutFull);
            if (!ok) break;
          }
          if (a + 1 < p.atoms) {
            mma_i8_lohi<1>(d_tmem, a_lo, b_lo, desc_hi, idesc, acc);
            mma_i8_lohi<1>(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1u);
            mma_i8_lohi<1>(d_tmem, a_lo + 4, b_lo + 4, desc_hi, idesc, 1u);
            mma_i8_lohi<1>(d_tmem, a_lo + 6, b_lo + 6, desc_hi, idesc, 1u);
            acc = 1u;
          } else {
            for (int k = 0; k < p.last_ksteps; ++k) {
              mma_i8_lohi<1>(d_tmem, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc, acc);
              acc = 1u;
            }
          }
          tc_commit_1cta(smem_u32(&ctrl->empty[stage]));
          a_lo += kAtomBytes >> 4;
          b_lo += b_step;
          if (++stage == p.stages) { stage = 0; phase ^= 1; b_lo = b_lo0; }
        }
        if (!ok) break;
        HY3D_TRACE_EVENT(1, tr, 2, u - unit_lo);
        tc_commit_1cta(smem_u32(&ctrl->tmem_full[buf]));
        // Last unit of this token block in the CTA's range: the block may be overwritten once
        // these MMAs have read it.
        if (u + 1 == unit_hi || (u + 1) / p.n_tiles != m) tc_commit_1cta(smem_u32(&ctrl->a_empty[abuf]));
      }
    }
    __syncwarp();
  } else if (warp < 2 + kEpiWarps) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;            // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;        // which of the warps sharing that quarter
    const bool geglu = kEpi == HY3D_EPI_GEGLU;
    const int64_t ldo = geglu ? (p.N >> 1) : p.N;
    const uint32_t stage_buf = staging_base + static_cast<uint32_t>((warp - 2) * p.store_bufs) * kSlabBytes;
    float* wsb = wsb_all + (warp - 2) * 256;   // this warp's column scales (128) and bias (128)
    float* bsb = wsb + 128;
    constexpr int kAps = geglu ? 2 * kSlabCols : kSlabCols;   // accumulator columns per slab
    constexpr int kApsLog2 = geglu ? 6 : 5;
    const int nslab = p.block_n / kAps;
    // this warp's slabs: half, half + kEpiPerQuarter, ...
    const int nmine = nslab > half ? (nslab - half + kEpiPerQuarter - 1) / kEpiPerQuarter : 0;
    const int ncols = nmine * kAps;                                  // <= 128
    const int pend = p.store_bufs - 1;
    bool ok = true;
    int it = 0, blk = -1, prev_m = -1, sb = 0;
    float as = 0.0f;
    // Column scales and bias of every slab this warp will take from a tile: fetched one tile
    // ahead (the loads fly under the previous tile's slabs), staged once per tile.
    float wv[4], bv[4];
    auto fetch_cols = [&](int u) {
      const int n0 = (u % p.n_tiles) * p.block_n;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int idx = lane + 32 * t;
        const int n = n0 + ((half + kEpiPerQuarter * (idx >> kApsLog2)) << kApsLog2) + (idx & (kAps - 1));
        const bool in = u < unit_hi && idx < ncols && n < p.N;
        wv[t] = in ? load_scalar(p.w_scale, p.ws_dtype, n) : 0.0f;
        bv[t] = (in && p.bias) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
      }
    };
    fetch_cols(unit_lo);
    for (int u = unit_lo; u < unit_hi; ++u, ++it) {
      const int m = u / p.n_tiles;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = m * kTileM;
      const int n0 = (u - m * p.n_tiles) * p.block_n;
      if (ok) ok = mbar_wait(smem_u32(&ctrl->tmem_full[buf]), acc_phase, abort_flag,
                             kDevTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);   // also: every lane is done with the previous tile's scales
      if (!ok) continue;
      tc_fence_after_sync();
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        wsb[lane + 32 * t] = wv[t];
        bsb[lane + 32 * t] = bv[t];
      }
      __syncwarp();
      fetch_cols(u + 1);
      if (threadIdx.x == 64) HY3D_TRACE_EVENT(2, tr, 3, u - unit_lo);
      if (m != prev_m) {   // the block's scales were published before its first MMA was issued
        prev_m = m;
        ++blk;
        as = ctrl->as[blk & (kScaleSlots - 1)][quarter * 32 + lane];
      }
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * p.acc_cols);
      const int out_row = m0 + quarter * 32;
      const bool rows_in = out_row < p.M;
      bool arrived = false;
      if (!geglu) {
        // 16-column chunks, two per slab; the tensor-memory load of chunk c+1 is in flight
        // while chunk c is rescaled, packed and written to the staging buffer.
        const int nchunk = 2 * nmine;
        uint32_t ra[16], rb[16];
        auto chunk_col = [&](int c) { return ((half + (c >> 1) * kEpiPerQuarter) << 5) + ((c & 1) << 4); };
        if (nchunk > 0) tmem_ld_x16(t_row + chunk_col(0), ra);
        for (int c = 0; c < nchunk; c += 2) {
          // ---- first half of a slab (registers ra) ----
          tmem_ld_wait();
          tmem_ld_x16(t_row + chunk_col(c + 1), rb);
          const uint32_t sbuf = stage_buf + sb * kSlabBytes;
          if (lane == 0) { if (pend) tma_store_wait_read<1>(); else tma_store_wait_read<0>(); }
          __syncwarp();
          chunk_math_store<kBf16, kEpi>(ra, as, wsb + (c << 4), bsb + (c << 4), sbuf, lane, 0);
          // ---- second half (registers rb) ----
          tmem_ld_wait();
          if (c + 2 < nchunk) {
            tmem_ld_x16(t_row + chunk_col(c + 2), ra);
          } else {
            // every accumulator column of this warp is in registers: hand the buffer back
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->tmem_empty[buf]));
            arrived = true;
          }
          chunk_math_store<kBf16, kEpi>(rb, as, wsb + (c << 4) + 16, bsb + (c << 4) + 16, sbuf, lane, 1);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int out_col = n0 + chunk_col(c);
            if (rows_in && out_col < p.N) tma_store_2d(&tm_o, sbuf, out_col * 2, out_row);
            tma_store_commit();
          }
          sb = (sb + 1) & pend;   // store_bufs is 1 or 2
        }
      } else {
        int j = 0;
        for (int s = half; s < nslab; s += kEpiPerQuarter, ++j) {
          uint32_t packed[16];
          const bool last = s + kEpiPerQuarter >= nslab;
          const int c0 = s * kAps;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            uint32_t rv[16], rg[16];
            tmem_ld_x16(t_row + c0 + 32 * b, rv);
            tmem_ld_x16(t_row + c0 + 32 * b + 16, rg);
            tmem_ld_wait();
            if (last && b == 1) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(&ctrl->tmem_empty[buf]));
              arrived = true;
            }
            dense::slab_math_geglu<kBf16>(rv, rg, as, wsb + j * kAps + 32 * b, bsb + j * kAps + 32 * b,
                                          packed + 8 * b);
          }
          const int out_col = (n0 + s * kAps) >> 1;
          dense::slab_store(packed, stage_buf + sb * kSlabBytes, lane, pend, &tm_o, out_col * 2, out_row,
                            rows_in && out_col < ldo);
          sb = (sb + 1) & pend;
        }
      }
      if (!arrived) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->tmem_empty[buf]));
      }
      if (threadIdx.x == 64) HY3D_TRACE_EVENT(2, tr, 4, u - unit_lo);
    }
    // Global writes of the bulk stores must be complete before the CTA retires.
    if (lane == 0) tma_store_wait_all<0>();
  } else {
    // ---------------- quantiser ----------------
    const int qw = warp - 2 - kEpiWarps;
    QuantCtx q;
    q.smem_base = smem_base;
    q.a_block_bytes = a_block_bytes;
    q.unit_lo = unit_lo;
    q.unit_hi = unit_hi;
    q.qw = qw;
    q.lane = lane;
    q.abort_flag = abort_flag;
    const int nvec = p.K >> 3;
    // Rows of 5 x 8, 5 x 16 or 5 x 32 vectors (K = 320, 640, 1280) run with the geometry
    // fixed at compile time; anything else takes the general loop.
    if (nvec == 5 * 8) quantiser_role<kBf16, 3, kRowsPerQuantWarp>(p, ctrl, q);
    else if (nvec == 5 * 16) quantiser_role<kBf16, 4, kRowsPerQuantWarp>(p, ctrl, q);
    else if (nvec == 5 * 32) quantiser_role<kBf16, 5, kRowsPerQuantWarp>(p, ctrl, q);
    else quantiser_role<kBf16, 0, kRowsPerQuantWarp>(p, ctrl, q);
    __syncwarp();
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
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_1cta(tmem_base, static_cast<uint32_t>(2 * p.acc_cols));
  }
}

}  // namespace

// Shape of a fused launch; filled by plan_fused.
struct FusedPlan {
  int block_n, n_tiles, m_blocks, atoms, a_bufs, store_bufs, stages, unit_align, grid, smem_bytes;
  int epi_warps;   // 8 or 16 of the 24 worker warps
};

// Whether the resident-block kernel can run this layer at all, and with which tiling.
// Returns HY3D_OK or the reason it cannot.
int plan_fused(int64_t M, int64_t N, int64_t K, int epilogue, int block_n, int sms, FusedPlan* plan) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 31) || (N & 15)) return HY3D_ERR_SHAPE;
  if (K > kMaxAtoms * 128) return HY3D_ERR_SHAPE;
  if (M > (1 << 30) || N > (1 << 30)) return HY3D_ERR_SHAPE;
  const bool geglu = epilogue == HY3D_EPI_GEGLU;
  if (geglu && (N & 31)) return HY3D_ERR_SHAPE;
  const int step = geglu ? 64 : 32;
  if (block_n != 0 && (block_n < step || block_n > 256 || block_n % step)) return HY3D_ERR_SHAPE;
  FusedPlan pl;
  pl.m_blocks = static_cast<int>((M + kTileM - 1) / kTileM);
  pl.atoms = static_cast<int>((K + 127) / 128);
  const int a_bytes = pl.atoms * kAtomBytes;
  // The epilogue handles N output columns per token, the quantiser K inputs, at about the
  // same cost per element: the wider side gets 16 of the 24 worker warps.
  const int kEpiWarps = (geglu ? N / 2 : N) >= K ? 16 : 8;
  pl.epi_warps = kEpiWarps;
  const int fixed0 = static_cast<int>(sizeof(FusedCtrl)) + kMaxEpiWarps * 256 * 4;
  // Shared-memory split for a tile width.  Preference: two resident blocks, then two staging
  // buffers per epilogue warp, as long as at least three weight stages remain; the deepest
  // rows get one block and what is left.
  auto fit = [&](int bn, FusedPlan& q) {
    const int b_bytes = bn * 128;
    const int tries[4][3] = {{2, 2, 3}, {2, 1, 3}, {1, 2, 3}, {1, 1, 2}};
    for (int t = 0; t < 4; ++t) {
      const int fixed = fixed0 + kEpiWarps * tries[t][1] * kSlabBytes + tries[t][0] * a_bytes;
      const int st = (kSmemLimit - fixed) / b_bytes;
      if (st >= tries[t][2]) {
        q.a_bufs = tries[t][0];
        q.store_bufs = tries[t][1];
        q.stages = st > kMaxStages ? kMaxStages : st;
        q.smem_bytes = fixed + q.stages * b_bytes;
        return true;
      }
    }
    return false;
  };
  if (block_n == 0) {
    // Cheapest tile width that fits: a tile costs its width plus a fixed overhead worth ~94
    // columns of MMA time (the dense kernel's model), so this minimises padded columns and the
    // number of tiles; a resident block that leaves little room narrows the tiles.
    const int lo = N <= 128 ? static_cast<int>((N + step - 1) / step * step) : 128;
    const int hi = N <= 128 ? lo : 256;
    int64_t best = -1;
    for (int bn = hi; bn >= lo; bn -= step) {
      FusedPlan q = pl;
      if (!fit(bn, q)) continue;
      const int64_t cost = ((N + bn - 1) / bn) * (bn + 94);
      if (best < 0 || cost < best) { best = cost; block_n = bn; }
    }
    if (best < 0) {   // nothing fits at 128 and above: take the widest narrower tile that does
      for (int bn = lo - step; bn >= step && block_n == 0; bn -= step) {
        FusedPlan q = pl;
        if (fit(bn, q)) block_n = bn;
      }
    }
    if (block_n == 0) return HY3D_ERR_SHAPE;
  }
  if (!fit(block_n, pl)) return HY3D_ERR_SHAPE;
  pl.block_n = block_n;
  pl.n_tiles = static_cast<int>((N + block_n - 1) / block_n);
  const int64_t total = static_cast<int64_t>(pl.m_blocks) * pl.n_tiles;
  pl.grid = static_cast<int>(total < sms ? total : sms);
  // Whole token blocks per CTA unless that leaves the last round of blocks badly filled or
  // there are fewer blocks than CTAs; then ranges are balanced to single units and a block
  // shared by two CTAs is quantised by both.
  pl.unit_align = pl.n_tiles;
  if (pl.m_blocks < sms) {
    pl.unit_align = 1;
  } else if (pl.n_tiles >= 4) {
    const int rounds = (pl.m_blocks + sms - 1) / sms;
    if (static_cast<int64_t>(rounds) * sms * 100 > static_cast<int64_t>(pl.m_blocks) * 112) pl.unit_align = 1;
  }
  if (pl.unit_align == pl.n_tiles) pl.grid = pl.m_blocks < sms ? pl.m_blocks : sms;
  *plan = pl;
  return HY3D_OK;
}

}  // namespace fused

// Which path hy3d_linear_w8a8_dense takes for a shape: 1 = the one-launch kernel of this file,
// 0 = quantise kernel + GEMM kernel.  Measured on B200 the one-launch kernel does not beat
// the two launches on any shape of the texture UNet (its 24 worker warps run the quantiser's
// and the epilogue's ~11 instructions per element at ~7 cycles per instruction per warp,
// while the stand-alone quantiser has 32 warps per SM to hide that latency), so the answer is
// 0 for every shape; the kernel stays available through hy3d_linear_w8a8_dense_fused.
int linear_path(int64_t M, int64_t K, int64_t N, int epilogue) {
  (void)M; (void)K; (void)N; (void)epilogue;
  return 0;
}

// Dense linear layer in one launch (see the file header).  x_dtype must equal out_dtype.
int linear_fused(const void* x, int x_dtype, int64_t ldx, float* scale_out, const int8_t* B,
                 const void* w_scale, int ws_dtype, const void* bias, int bias_dtype, void* out,
                 int out_dtype, int64_t M, int64_t N, int64_t K, int epilogue, int block_n,
                 cudaStream_t stream) {
  using namespace fused;
  if (x_dtype != HY3D_F16 && x_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if (out_dtype != x_dtype) return HY3D_ERR_ARG;
  if (epilogue < HY3D_EPI_LINEAR || epilogue > HY3D_EPI_GEGLU) return HY3D_ERR_ARG;
  if (ws_dtype < HY3D_F16 || ws_dtype > HY3D_F32) return HY3D_ERR_ARG;
  if (bias && (bias_dtype < HY3D_F16 || bias_dtype > HY3D_F32)) return HY3D_ERR_ARG;
  if (M < 0) return HY3D_ERR_SHAPE;
  if (M == 0) return (N > 0 && K > 0) ? HY3D_OK : HY3D_ERR_SHAPE;
  if (!x || !B || !out || !w_scale) return HY3D_ERR_ARG;
  if (ldx < K || (ldx & 7)) return HY3D_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return HY3D_ERR_SHAPE;
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  FusedPlan pl;
  int rc = plan_fused(M, N, K, epilogue, block_n, sms, &pl);
  if (rc != HY3D_OK) return rc;

  FusedArgs p;
  p.x = static_cast<const uint16_t*>(x);
  p.ldx = ldx;
  p.scale_out = scale_out;
  p.w_scale = w_scale; p.bias = bias; p.ws_dtype = ws_dtype; p.bias_dtype = bias_dtype;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.block_n = pl.block_n; p.stages = pl.stages; p.store_bufs = pl.store_bufs;
  int acc_cols = 32;
  while (acc_cols < pl.block_n) acc_cols <<= 1;
  p.acc_cols = acc_cols;
  p.m_blocks = pl.m_blocks; p.n_tiles = pl.n_tiles; p.atoms = pl.atoms;
  p.last_ksteps = static_cast<int>((K - static_cast<int64_t>(pl.atoms - 1) * 128) / 32);
  p.a_bufs = pl.a_bufs;
  p.unit_align = pl.unit_align;
  // Lanes per row: the power of two (4..32) that leaves at most five 16-byte vectors per lane.
  const int nvec = static_cast<int>(K >> 3);
  int lg = 2;   // at most 8 rows per batch, so a batch fits the rows of one quantiser warp
  while (lg < 5 && (nvec + (1 << lg) - 1) / (1 << lg) > kMaxVecs) ++lg;
  p.q_lanes_log2 = lg;
  p.q_vecs = (nvec + (1 << lg) - 1) >> lg;
  if (p.q_vecs > kMaxVecs) return HY3D_ERR_SHAPE;
  p.debug = 0;
#ifdef HY3D_TRACE
  { const char* e = getenv("HY3D_DEBUG"); p.debug = e ? atoi(e) : 0; }
#endif

  const bool geglu = epilogue == HY3D_EPI_GEGLU;
  CUtensorMap tm_b, tm_o;
  rc = encode_tmap_2d_u8(&tm_b, B, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                         static_cast<uint64_t>(K), 128, static_cast<uint32_t>(pl.block_n), 128);
  if (rc != HY3D_OK) return rc;
  const uint64_t row_bytes = static_cast<uint64_t>(geglu ? N / 2 : N) * 2;
  rc = encode_tmap_2d_u8(&tm_o, out, row_bytes, static_cast<uint64_t>(M), row_bytes, kSlabCols * 2, 32, 64);
  if (rc != HY3D_OK) return rc;

  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const FusedArgs);
#define HY3D_FUSED_ROW(EW)                                                                            \
  {{linear_fused_kernel<false, HY3D_EPI_LINEAR, EW>, linear_fused_kernel<false, HY3D_EPI_GELU, EW>,   \
    linear_fused_kernel<false, HY3D_EPI_GEGLU, EW>},                                                  \
   {linear_fused_kernel<true, HY3D_EPI_LINEAR, EW>, linear_fused_kernel<true, HY3D_EPI_GELU, EW>,     \
    linear_fused_kernel<true, HY3D_EPI_GEGLU, EW>}}
  static const KernelFn kernels[2][2][3] = {HY3D_FUSED_ROW(8), HY3D_FUSED_ROW(16)};
#undef HY3D_FUSED_ROW
  const int ki = x_dtype == HY3D_BF16 ? 1 : 0;
  const KernelFn kernel = kernels[pl.epi_warps == 16 ? 1 : 0][ki][epilogue];
  rc = ensure_max_smem(reinterpret_cast<const void*>(kernel), kSmemLimit);
  if (rc != HY3D_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pl.grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(pl.smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1] = {pdl_attribute()};
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, tm_b, tm_o, p) != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace hy3d
