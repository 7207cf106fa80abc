// Weight-stationary-in-M GEMM family for sm_100a:  D[feature, token] = W[feature, :] . X[token, :]
//
// Every linear layer of the engine goes through this one kernel.  The weight matrix
// (nn.Linear layout [out_features, in_features], i.e. K-major) is the tcgen05 A operand
// with a fixed 128-row tile; the activations [tokens, in_features] (also K-major) are the
// B operand with a token tile BN in {16, 32, 64, 128, 256}.  A decode step with a handful
// of tokens therefore issues the same 128 x BN x 16 UMMA as a 2048-token prefill chunk;
// only BN, split-K and the pipeline depth change.  Both operands are staged by TMA
// (cp.async.bulk.tensor.2d, 128-byte swizzle, no cluster qualifier) into a ring of
// shared-memory stages; one elected thread issues tcgen05.mma into a TMEM accumulator and
// four epilogue warps read it back with tcgen05.ld.
//
// Epilogues: bias (per feature), GELU (tanh or erf), residual add, bf16 store
// out[token][feature]; fp32 split-K partials part[split][token][feature]; and the dual
// form (two weight tiles per stage, two accumulators) that writes
// silu(gate) * up directly, which replaces the reference's CUTLASS DualGemm
// (prism_infer/ops/csrc/cutlass_dual_gemm_swiglu.cu:85-215, mma.sync Sm80) and every
// F.linear of prism_infer/layers/linear.py:62-190.
//
// Programmatic dependent launch: the producer thread prefetches the first ring of weight
// tiles (which never depend on the previous kernel) before griddepcontrol.wait, then
// loads activations.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

PRISM_DEFINE_TU_STATUS(gemm)

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_LIMIT = 232448;  // 227 KB

struct GemmArgs {
  int M;             // valid weight rows (features)
  int T;             // valid tokens
  int kb_total;      // ceil(K / 64)
  int kb_per_split;  // k-blocks handled by one blockIdx.z
  int w2_row_off;    // dual: first row of the second weight matrix inside the same tensor map
  int stages;
  int tokens_fastest;  // grid rasterisation, see the kernel
  int out_f32;       // 1: fp32 partial output, one slab per split
  int act;           // 0 none, 1 gelu(tanh), 2 gelu(erf)
  long long ldo;     // output row stride (elements)
  long long ldr;     // residual row stride (elements)
  long long split_stride;  // elements between split slabs
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  void* out;
  // push mode (tensor parallel, fused GEMM -> exchange): the fp32 partial tile is written
  // into every rank's slab group and the last CTA raises a flag on every rank.
  int n_peers;               // 0 = off
  int my_rank;
  int push_rows;             // 1: all-gather form, bf16 rows [row_base + token] on every rank
  long long row_base;
  long long point;           // exchange point inside the step (or an absolute sequence number)
  int* cta_counter;          // local, zero-initialised, self-resetting
  const unsigned long long* epoch;  // local device word: sequence base of the current step (null: 0)
  float* peer_out[8];        // slab buffers (or bf16 row buffers) of this slot on every rank (incl. own)
  unsigned long long* peer_flag[8];  // flag arrays [tp] of this slot on every rank
};

template <int BN, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmArgs a) {
  constexpr int X_TILE_BYTES = BN * BK * 2;
  constexpr int W_STAGE_BYTES = W_TILE_BYTES * (DUAL ? 2 : 1);
  constexpr int STAGE_BYTES = W_STAGE_BYTES + X_TILE_BYTES;
  constexpr int ACC_COLS = DUAL ? 2 * BN : BN;
  constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;  // power of two by construction
  constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = a.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* tmem_full = empty + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Rasterisation.  When the weight matrix does not fit the 126 MB L2, token tiles vary
  // fastest so the CTAs that share a weight tile run together and it leaves DRAM once;
  // otherwise feature tiles vary fastest (measured faster while everything is L2-resident).
  const int m0 = (a.tokens_fastest ? blockIdx.y : blockIdx.x) * BM;
  const int n0 = (a.tokens_fastest ? blockIdx.x : blockIdx.y) * BN;
  const int split = blockIdx.z;
  const int kb_begin = split * a.kb_per_split;
  const int kb_end = min(a.kb_total, kb_begin + a.kb_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);  // the TMA transaction
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      const int pre = min(stages, num_kb);
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + (size_t)i * STAGE_BYTES;
        mbar_expect_tx(&full[i], STAGE_BYTES);
        tma_load_2d(st, &tmW, &full[i], (kb_begin + i) * BK, m0);
        if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, &full[i], (kb_begin + i) * BK, a.w2_row_off + m0);
      }
      pdl_wait();  // activations come from the previous kernel
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + (size_t)i * STAGE_BYTES;
        tma_load_2d(st + W_STAGE_BYTES, &tmX, &full[i], (kb_begin + i) * BK, n0);
      }
      int issued = pre;
      bool ok = true;
      for (int kb = pre; kb < num_kb && ok; ++kb) {
        const int s = kb % stages;
        const uint32_t round = kb / stages;
        ok = mbar_wait(&empty[s], (round - 1) & 1, 1);
        if (!ok) break;
        uint8_t* st = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(st, &tmW, &full[s], (kb_begin + kb) * BK, m0);
        if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, &full[s], (kb_begin + kb) * BK, a.w2_row_off + m0);
        tma_load_2d(st + W_STAGE_BYTES, &tmX, &full[s], (kb_begin + kb) * BK, n0);
        issued = kb + 1;
      }
      if (!ok) {
        // Unwinding after a timed-out wait: let copies already in flight land before the
        // CTA's shared memory is released.
        for (int kb = max(0, issued - stages); kb < issued; ++kb) {
          (void)mbar_wait(&full[kb % stages], (kb / stages) & 1, 4);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------ MMA issuer ------------------------------
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % stages;
        ok = mbar_wait(&full[s], (kb / stages) & 1, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t da = umma_desc_sw128(st);
        const uint64_t db = umma_desc_sw128(st + W_STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t acc = (kb | k) != 0;
          tc_mma_f16(tmem_base, da + 2 * k, db + 2 * k, IDESC, acc);
          if (DUAL) {
            const uint64_t da2 = umma_desc_sw128(st + W_TILE_BYTES);
            tc_mma_f16(tmem_base + BN, da2 + 2 * k, db + 2 * k, IDESC, acc);
          }
        }
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(tmem_full);
    }
  } else {
    // ------------------------------ epilogue warps 2..5 ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    pdl_wait();
    if (mbar_wait(tmem_full, 0, 3)) {
      tc_fence_after();
      const int m = m0 + q * 32 + lane;
      const bool m_ok = m < a.M;
      const float bias_v = (a.bias != nullptr && m_ok) ? __bfloat162float(a.bias[m]) : 0.0f;
      const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
      float* out_f = reinterpret_cast<float*>(a.out) + (size_t)split * a.split_stride;
      __nv_bfloat16* out_b = reinterpret_cast<__nv_bfloat16*>(a.out);
      // One compact store loop per output form; the form is chosen once, outside the column
      // loops, so the instruction stream of a tile touches only the code it needs.
      enum { EPI_BF16_PLAIN, EPI_BF16_FULL, EPI_F32, EPI_PUSH_F32, EPI_PUSH_ROWS, EPI_DUAL };
      int mode;
      if (DUAL) mode = EPI_DUAL;
      else if (a.n_peers > 0) mode = a.push_rows ? EPI_PUSH_ROWS : EPI_PUSH_F32;
      else if (a.out_f32) mode = EPI_F32;
      else mode = (a.bias == nullptr && a.act == 0 && a.residual == nullptr) ? EPI_BF16_PLAIN : EPI_BF16_FULL;
      const int n_valid = min(BN, a.T - n0);
      unsigned long long push_seq = 0;
      if (mode == EPI_PUSH_F32)
        push_seq = (((a.epoch ? *a.epoch : 0ull) + (unsigned long long)a.point) & 0xffffffffull) << 32;
      for (int c0 = 0; c0 < n_valid; c0 += 16) {
        uint32_t r[16];
        uint32_t r2[16];
        tmem_ld16(t_lane + c0, r);
        if (DUAL) tmem_ld16(t_lane + BN + c0, r2);
        tmem_ld_wait();
        if (!m_ok) continue;
        const int cols = min(16, n_valid - c0);
        const size_t row0 = (size_t)(n0 + c0);
        switch (mode) {
          case EPI_BF16_PLAIN: {
            __nv_bfloat16* dst = out_b + row0 * a.ldo + m;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < cols) dst[(size_t)j * a.ldo] = __float2bfloat16_rn(__uint_as_float(r[j]));
            break;
          }
          case EPI_BF16_FULL: {
            __nv_bfloat16* dst = out_b + row0 * a.ldo + m;
            const __nv_bfloat16* rsd = a.residual ? a.residual + row0 * a.ldr + m : nullptr;
            // all residual loads first: out may alias residual (in-place add), and loads that
            // sit between the stores would each wait for the store before them
            float res[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) res[j] = (rsd != nullptr && j < cols) ? __bfloat162float(rsd[(size_t)j * a.ldr]) : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < cols) {
                float v = __uint_as_float(r[j]) + bias_v;
                if (a.act == 1) v = gelu_tanh(v);
                else if (a.act == 2) v = gelu_erf(v);
                if (rsd != nullptr) v = bf16_round(v) + res[j];
                dst[(size_t)j * a.ldo] = __float2bfloat16_rn(v);
              }
            }
            break;
          }
          case EPI_F32: {
            float* dst = out_f + row0 * a.ldo + m;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < cols) dst[(size_t)j * a.ldo] = __uint_as_float(r[j]);
            break;
          }
          case EPI_PUSH_F32: {
            // one 8-byte store per element: fp32 value in the low half, the exchange's sequence
            // number in the high half.  An aligned 8-byte store is single-copy atomic, so a
            // consumer that sees the expected sequence number also sees the value; no fence,
            // counter or flag is needed on this path.
            const size_t off = (size_t)(a.my_rank * (int)gridDim.z + split) * a.split_stride + row0 * a.ldo + m;
            for (int p = 0; p < a.n_peers; ++p) {
              unsigned long long* dst = reinterpret_cast<unsigned long long*>(a.peer_out[p]) + off;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (j < cols) {
                  const unsigned long long word = push_seq | (unsigned long long)r[j];
                  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + (size_t)j * a.ldo), "l"(word) : "memory");
                }
              }
            }
            break;
          }
          case EPI_PUSH_ROWS: {
            // fused GEMM -> all-gather: this rank's rows land in every rank's copy
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = __uint_as_float(r[j]) + bias_v;
              if (a.act == 1) v = gelu_tanh(v);
              else if (a.act == 2) v = gelu_erf(v);
              packed[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
            }
            const size_t off = (size_t)(a.row_base + row0) * a.ldo + m;
            for (int p = 0; p < a.n_peers; ++p) {
              unsigned short* dst = reinterpret_cast<unsigned short*>(a.peer_out[p]) + off;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (j < cols) dst[(size_t)j * a.ldo] = (unsigned short)packed[j];
            }
            break;
          }
          default: {  // EPI_DUAL: silu(gate) -> bf16, * up -> bf16 (rounding points of the eager graph)
            __nv_bfloat16* dst = out_b + row0 * a.ldo + m;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < cols) {
                const float g = bf16_round(__uint_as_float(r[j]));
                const float u = bf16_round(__uint_as_float(r2[j]));
                dst[(size_t)j * a.ldo] = __float2bfloat16_rn(bf16_round(silu(g)) * u);
              }
            }
            break;
          }
        }
      }
    }
  }
  const bool flagged = a.n_peers > 0 && a.push_rows;  // the all-gather form signals with flags
  if (flagged && warp >= 2) __threadfence_system();  // this CTA's rows visible to every GPU
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (flagged && threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y * gridDim.z;
    const int old = atomicAdd(a.cta_counter, 1);
    if (old == total - 1) {
      *a.cta_counter = 0;
      __threadfence_system();
      // one fence above, then plain posted stores: a release store per peer would serialise
      // one NVLink round trip per peer
      const unsigned long long seq = (a.epoch ? *a.epoch : 0ull) + (unsigned long long)a.point;
      for (int p = 0; p < a.n_peers; ++p) {
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[p] + a.my_rank), "l"(seq) : "memory");
      }
    }
  }
}


// ------------------------------------------------------------------------------------
// Persistent form for prefill-sized problems (no split-K, bf16 output): one CTA per SM walks
// a strided list of output tiles.  The TMA producer runs ahead across tile boundaries, the
// MMA thread alternates between two TMEM accumulators when both fit (BN * (DUAL ? 2 : 1)
// <= 256 columns), and the epilogue warps drain one accumulator while the next tile's MMAs
// run, so tile set-up, pipeline fill and the store loop are off the tensor pipe's critical
// path.
// ------------------------------------------------------------------------------------
struct PersistArgs {
  int dual_rm;  // row-major form only: the B tile is 128 gate rows followed by 128 up rows, epilogue = SwiGLU
  int M, T, kb_total, w2_row_off, stages;
  int m_tiles, n_tiles;
  int tokens_fastest;
  int act;
  long long ldo, ldr;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  // scatter form (row-major only; fused row-parallel GEMM -> reduce-scatter): token row m belongs
  // to rank m / rows_per_owner and is written into that rank's buffer, slab my_rank, as bf16; when
  // every CTA is done flag[my_rank] on every rank is set to seq.
  int scatter;
  int rows_per_owner;
  int n_peers, my_rank;
  unsigned long long seq;
  const unsigned long long* epoch;  // when set, the flag value is *epoch + seq (graph replays advance the epoch)
  int* cta_counter;
  __nv_bfloat16* peer_out[8];
  unsigned long long* peer_flag[8];
};

// ROWMAJOR: the A operand (128-row tiles, TMEM lanes) holds the tokens and B the weights, so an
// epilogue thread owns one token row and 16 consecutive features per TMEM load: bias, residual
// and output move as 16-byte vectors instead of sixteen strided 2-byte accesses (the strided
// residual loads made the vision projections 6x slower than their main loop).  In that form
// a.M counts tokens and a.T features.
template <int BN, bool DUAL, bool ROWMAJOR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_wx_persistent_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                          const PersistArgs a) {
  constexpr int X_TILE_BYTES = BN * BK * 2;
  constexpr int W_STAGE_BYTES = W_TILE_BYTES * (DUAL ? 2 : 1);
  constexpr int STAGE_BYTES = W_STAGE_BYTES + X_TILE_BYTES;
  constexpr int ACC_COLS = DUAL ? 2 * BN : BN;
  constexpr int NBUF = ACC_COLS * 2 <= 512 ? 2 : 1;
  constexpr int TMEM_COLS = ACC_COLS * NBUF < 32 ? 32 : ACC_COLS * NBUF;
  constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = a.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;   // [NBUF] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;    // [NBUF] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = a.m_tiles * a.n_tiles;
  const int num_kb = a.kb_total;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  // tile id -> (m0, n0); consecutive ids share a weight tile (tokens fastest) or an
  // activation tile (features fastest)
#define PRISM_TILE_COORDS(tile_, m0_, n0_)                                             \
  const int m0_ = (a.tokens_fastest ? (tile_) / a.n_tiles : (tile_) % a.m_tiles) * BM; \
  const int n0_ = (a.tokens_fastest ? (tile_) % a.n_tiles : (tile_) / a.m_tiles) * BN;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      pdl_wait();  // activations come from the previous kernel
      long long it = 0;  // running k-block count across tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        PRISM_TILE_COORDS(tile, m0, n0)
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % stages);
          const uint32_t round = (uint32_t)(it / stages);
          if (round > 0) {
            ok = mbar_wait(&empty[s], (round - 1) & 1, 1);
            if (!ok) break;
          }
          uint8_t* st = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(st, &tmW, &full[s], kb * BK, m0);
          if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, &full[s], kb * BK, a.w2_row_off + m0);
          if (ROWMAJOR && a.dual_rm) {
            // one 256-row B tile made of 128 gate rows and the matching 128 up rows
            tma_load_2d(st + W_STAGE_BYTES, &tmX, &full[s], kb * BK, n0 / 2);
            tma_load_2d(st + W_STAGE_BYTES + X_TILE_BYTES / 2, &tmX, &full[s], kb * BK, a.w2_row_off + n0 / 2);
          } else {
            tma_load_2d(st + W_STAGE_BYTES, &tmX, &full[s], kb * BK, n0);
          }
        }
      }
      if (!ok) {
        // unwinding after a timed-out wait: let copies already in flight land before the
        // CTA's shared memory is released
        for (long long j = it - stages < 0 ? 0 : it - stages; j < it; ++j)
          (void)mbar_wait(&full[j % stages], (uint32_t)(j / stages) & 1, 4);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------ MMA issuer ------------------------------
      long long it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local % NBUF;
        const uint32_t use = (uint32_t)(local / NBUF);
        if (use > 0) {
          ok = mbar_wait(&acc_empty[buf], (use - 1) & 1, 5);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % stages);
          ok = mbar_wait(&full[s], (uint32_t)(it / stages) & 1, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(st);
          const uint64_t db = umma_desc_sw128(st + W_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t acc = (kb | k) != 0;
            tc_mma_f16(acc_addr, da + 2 * k, db + 2 * k, IDESC, acc);
            if (DUAL) {
              const uint64_t da2 = umma_desc_sw128(st + W_TILE_BYTES);
              tc_mma_f16(acc_addr + BN, da2 + 2 * k, db + 2 * k, IDESC, acc);
            }
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue warps 2..5 ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    pdl_wait();
    const bool plain = !DUAL && a.bias == nullptr && a.act == 0 && a.residual == nullptr;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local % NBUF;
      if (!mbar_wait(&acc_full[buf], (uint32_t)(local / NBUF) & 1, 3)) break;
      tc_fence_after();
      PRISM_TILE_COORDS(tile, m0, n0)
      const int m = m0 + q * 32 + lane;
      const bool m_ok = m < a.M;
      const uint32_t t_lane = tmem_base + buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
      const int n_valid = min(BN, a.T - n0);
      if (ROWMAJOR && a.dual_rm) {
        // lane = token m; accumulator columns 0..127 = gate features n0/2 + c, 128..255 = up
        const int f_base = n0 / 2;
        const int f_valid = min(BN / 2, a.T / 2 - f_base);
        for (int c0 = 0; c0 < f_valid; c0 += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld16(t_lane + c0, rg);
          tmem_ld16(t_lane + BN / 2 + c0, ru);
          tmem_ld_wait();
          if (!m_ok) continue;
          uint4 o[2];
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float g0 = bf16_round(__uint_as_float(rg[2 * e])), g1 = bf16_round(__uint_as_float(rg[2 * e + 1]));
            const float u0 = bf16_round(__uint_as_float(ru[2 * e])), u1 = bf16_round(__uint_as_float(ru[2 * e + 1]));
            op[e] = __floats2bfloat162_rn(bf16_round(silu(g0)) * u0, bf16_round(silu(g1)) * u1);
          }
          __nv_bfloat16* dst = a.out + (size_t)m * a.ldo + f_base + c0;
          *reinterpret_cast<uint4*>(dst) = o[0];
          *reinterpret_cast<uint4*>(dst + 8) = o[1];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        continue;
      }
      if (ROWMAJOR) {
        // lane = token m, columns = features n0 + c0 .. + 15 (a.T is a multiple of 16 here)
        for (int c0 = 0; c0 < n_valid; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(t_lane + c0, r);
          tmem_ld_wait();
          if (!m_ok) continue;
          const int f0 = n0 + c0;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
          if (a.bias != nullptr) {
            const uint4 b0 = *reinterpret_cast<const uint4*>(a.bias + f0), b1 = *reinterpret_cast<const uint4*>(a.bias + f0 + 8);
            const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&b0);
            const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&b1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x0 = __bfloat1622float2(p0[e]), x1 = __bfloat1622float2(p1[e]);
              v[2 * e] += x0.x;
              v[2 * e + 1] += x0.y;
              v[8 + 2 * e] += x1.x;
              v[8 + 2 * e + 1] += x1.y;
            }
          }
          if (a.act == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_tanh(v[j]);
          } else if (a.act == 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_erf(v[j]);
          }
          if (a.residual != nullptr) {
            const __nv_bfloat16* rs = a.residual + (size_t)m * a.ldr + f0;
            const uint4 r0 = *reinterpret_cast<const uint4*>(rs), r1 = *reinterpret_cast<const uint4*>(rs + 8);
            const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
            const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x0 = __bfloat1622float2(p0[e]), x1 = __bfloat1622float2(p1[e]);
              v[2 * e] = bf16_round(v[2 * e]) + x0.x;
              v[2 * e + 1] = bf16_round(v[2 * e + 1]) + x0.y;
              v[8 + 2 * e] = bf16_round(v[8 + 2 * e]) + x1.x;
              v[8 + 2 * e + 1] = bf16_round(v[8 + 2 * e + 1]) + x1.y;
            }
          }
          uint4 o[2];
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
          for (int e = 0; e < 8; ++e) op[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
          __nv_bfloat16* dst;
          if (a.scatter) {
            const int owner = m / a.rows_per_owner;
            dst = a.peer_out[owner] + ((size_t)a.my_rank * a.rows_per_owner + (m - owner * a.rows_per_owner)) * a.ldo + f0;
          } else {
            dst = a.out + (size_t)m * a.ldo + f0;
          }
          *reinterpret_cast<uint4*>(dst) = o[0];
          *reinterpret_cast<uint4*>(dst + 8) = o[1];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        continue;
      }
      const float bias_v = (a.bias != nullptr && m_ok) ? __bfloat162float(a.bias[m]) : 0.0f;
      for (int c0 = 0; c0 < n_valid; c0 += 16) {
        uint32_t r[16];
        uint32_t r2[16];
        tmem_ld16(t_lane + c0, r);
        if (DUAL) tmem_ld16(t_lane + BN + c0, r2);
        tmem_ld_wait();
        if (!m_ok) continue;
        const int cols = min(16, n_valid - c0);
        const size_t row0 = (size_t)(n0 + c0);
        __nv_bfloat16* dst = a.out + row0 * a.ldo + m;
        if (DUAL) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < cols) {
              const float g = bf16_round(__uint_as_float(r[j]));
              const float u = bf16_round(__uint_as_float(r2[j]));
              dst[(size_t)j * a.ldo] = __float2bfloat16_rn(bf16_round(silu(g)) * u);
            }
          }
        } else if (plain) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < cols) dst[(size_t)j * a.ldo] = __float2bfloat16_rn(__uint_as_float(r[j]));
        } else {
          const __nv_bfloat16* rsd = a.residual ? a.residual + row0 * a.ldr + m : nullptr;
          // all residual loads first: out may alias residual (in-place add), and loads that sit
          // between the stores would each wait for the store before them
          float res[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) res[j] = (rsd != nullptr && j < cols) ? __bfloat162float(rsd[(size_t)j * a.ldr]) : 0.0f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < cols) {
              float v = __uint_as_float(r[j]) + bias_v;
              if (a.act == 1) v = gelu_tanh(v);
              else if (a.act == 2) v = gelu_erf(v);
              if (rsd != nullptr) v = bf16_round(v) + res[j];
              dst[(size_t)j * a.ldo] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      // this warp's reads of the accumulator are complete: hand the buffer back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
#undef PRISM_TILE_COORDS
  if (ROWMAJOR && a.scatter && warp >= 2) __threadfence_system();  // this CTA's rows visible to their owners
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (ROWMAJOR && a.scatter && threadIdx.x == 0) {
    const int old = atomicAdd(a.cta_counter, 1);
    if (old == (int)gridDim.x - 1) {
      *a.cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < a.n_peers; ++p)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer_flag[p] + a.my_rank), "l"((a.epoch ? *a.epoch : 0ull) + a.seq) : "memory");
    }
  }
}

// ------------------------------------------------------------------------------------
// Host side: tensor-map cache and launcher.
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  unsigned long long rows, cols, ld;
  unsigned box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= k.ld * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    h ^= k.box_rows * 0x27D4EB2F165667C5ull;
    return h;
  }
};

std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// A [rows, cols] bf16 row-major matrix with row stride ld (elements); box = box_rows x 64.
int get_tensor_map(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                   unsigned box_rows, CUtensorMap* out) {
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -100;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return -101;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -102 - (int)r;
  if (g_maps.size() > 65536) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return 0;
}

int g_small_tile_smem_cap = 0;

template <int BN, bool DUAL>
int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, GemmArgs& a, int m_tiles, int splits, int stages_override,
                cudaStream_t stream, bool pdl) {
  constexpr int STAGE_BYTES = W_TILE_BYTES * (DUAL ? 2 : 1) + BN * BK * 2;
  int max_stages = (SMEM_LIMIT - 1024 - 512) / STAGE_BYTES;
  if (max_stages > 16) max_stages = 16;
  if (BN <= 32 && g_small_tile_smem_cap > 0) {
    // decode-sized launches: leave room for the next kernel's CTA on the same SM, so that its
    // weight prefetch (issued before griddepcontrol.wait) overlaps this kernel's tail
    int capped = (g_small_tile_smem_cap - 1024 - 512) / STAGE_BYTES;
    if (capped < 2) capped = 2;
    if (capped < max_stages) max_stages = capped;
  }
  int stages = stages_override > 0 ? min(stages_override, max_stages) : max_stages;
  if (stages > a.kb_per_split) stages = a.kb_per_split;
  if (stages < 1) stages = 1;
  a.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + (2 * stages + 1) * 8 + 48;
  static int configured_smem = 0;
  if ((int)smem > configured_smem) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wx_kernel<BN, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) return (int)e;
    configured_smem = SMEM_LIMIT;
  }
  const int n_tiles = (a.T + BN - 1) / BN;
  dim3 grid = a.tokens_fastest ? dim3(n_tiles, m_tiles, splits) : dim3(m_tiles, n_tiles, splits);
  cudaError_t e = prism_launch(gemm_wx_kernel<BN, DUAL>, grid, dim3(GEMM_THREADS), smem, stream, pdl, tw, tx, a);
  return (int)e;
}


int g_persistent_min_tokens = 512;  // 0 disables the persistent form
int g_persistent_rowmajor = 1;      // 1: tokens on the TMEM lanes for the non-dual persistent GEMM
int g_sm_count = 0;

template <int BN, bool DUAL, bool ROWMAJOR = false>
int launch_persistent(const CUtensorMap& tw, const CUtensorMap& tx, PersistArgs& a, cudaStream_t stream, bool pdl) {
  constexpr int STAGE_BYTES = W_TILE_BYTES * (DUAL ? 2 : 1) + BN * BK * 2;
  int stages = (SMEM_LIMIT - 1024 - 512) / STAGE_BYTES;
  if (stages > 12) stages = 12;
  if (stages < 2) return -7;
  a.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + (2 * stages + 4) * 8 + 64;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wx_persistent_kernel<BN, DUAL, ROWMAJOR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (g_sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      g_sm_count = 148;
  }
  const int tiles = a.m_tiles * a.n_tiles;
  const int grid = tiles < g_sm_count ? tiles : g_sm_count;
  return (int)prism_launch(gemm_wx_persistent_kernel<BN, DUAL, ROWMAJOR>, dim3(grid), dim3(GEMM_THREADS), smem, stream, pdl, tw, tx, a);
}

}  // namespace

int prism_get_tensor_map(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                         unsigned box_rows, CUtensorMap* out) {
  return get_tensor_map(ptr, rows, cols, ld, box_rows, out);
}

// [tokens][heads][head_dim] bf16 view (head stride = head_dim, token stride ld elements) with a
// box of box_rows tokens x 1 head x 64 columns, 128-byte swizzle.  Columns past head_dim are
// out of bounds of the innermost dimension and read as zeros, whatever the neighbouring head
// holds.  Not cached: the encode costs about a microsecond.
int prism_make_head_tensor_map(const void* ptr, unsigned long long tokens, unsigned heads, unsigned head_dim,
                               unsigned long long ld, unsigned box_rows, CUtensorMap* out) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -100;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15) || ((head_dim * 2) & 15)) return -101;
  cuuint64_t dims[3] = {head_dim, heads, tokens};
  cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, ld * 2};
  cuuint32_t box[3] = {BK, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -102 - (int)r;
}

// W [w_rows_total, K] (row stride ldw), X [T, K] (row stride ldx), both bf16.
// out: bf16 [T, ldo] (features along the row) or fp32 [splits][T][ldo] when out_f32.
// dual: second weight tile starts at row w2_row_off; output = silu(W1 x) * (W2 x), M rows.
// Returns 0 on success, a cudaError_t (>0) or a negative validation code.
struct PushSpec {
  int n_peers, my_rank, push_rows;
  long long point, row_base;
  int* cta_counter;
  const unsigned long long* epoch;
  float* peer_out[8];
  unsigned long long* peer_flag[8];
};

static int gemm_wx_impl(const void* W, const void* X, void* out, int M, int T, int K, long long ldw, long long ldx,
                        long long ldo, int w_rows_total, const void* bias, const void* residual, long long ldr, int act,
                        int dual, int w2_row_off, int splits, int out_f32, long long split_stride, int bn_override,
                        int stages_override, void* stream_ptr, int pdl, const PushSpec* push) {
  if (M <= 0 || T <= 0 || K <= 0) return -1;
  if (K % 8) return -2;  // 16-byte row pitch for TMA
  if (dual && (splits > 1 || out_f32)) return -3;
  if (!out_f32 && splits > 1) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  int bn = bn_override;
  if (bn <= 0) {
    if (T <= 16) bn = 16;
    else if (T <= 32) bn = 32;
    else if (T <= 64) bn = 64;
    else if (T <= 128) bn = 128;
    else {
      const int pad256 = (T + 255) / 256 * 256, pad128 = (T + 127) / 128 * 128;
      bn = (pad256 * 100 <= pad128 * 106) ? 256 : 128;
    }
  }
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return -5;
  GemmArgs a;
  a.M = M;
  a.T = T;
  a.kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > a.kb_total) splits = a.kb_total;
  a.kb_per_split = (a.kb_total + splits - 1) / splits;
  splits = (a.kb_total + a.kb_per_split - 1) / a.kb_per_split;  // no empty split
  a.w2_row_off = w2_row_off;
  a.stages = 0;
  a.tokens_fastest = ((long long)w_rows_total * K * 2 > (100ll << 20) || (M + BM - 1) / BM > 65535) ? 1 : 0;
  a.out_f32 = out_f32;
  a.act = act;
  a.ldo = ldo;
  a.ldr = ldr;
  a.split_stride = split_stride;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.out = out;
  a.n_peers = 0;
  a.my_rank = 0;
  a.point = 0;
  a.push_rows = 0;
  a.row_base = 0;
  a.cta_counter = nullptr;
  a.epoch = nullptr;
  for (int p = 0; p < 8; ++p) {
    a.peer_out[p] = nullptr;
    a.peer_flag[p] = nullptr;
  }
  if (push != nullptr) {
    a.n_peers = push->n_peers;
    a.my_rank = push->my_rank;
    a.point = push->point;
    a.push_rows = push->push_rows;
    a.row_base = push->row_base;
    a.cta_counter = push->cta_counter;
    a.epoch = push->epoch;
    for (int p = 0; p < push->n_peers && p < 8; ++p) {
      a.peer_out[p] = push->peer_out[p];
      a.peer_flag[p] = push->peer_flag[p];
    }
  }
  CUtensorMap tw, tx;
  int rc = get_tensor_map(W, (unsigned long long)w_rows_total, (unsigned long long)K, (unsigned long long)ldw, BM, &tw);
  if (rc) return rc;
  rc = get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, (unsigned)bn, &tx);
  if (rc) return rc;
  const int m_tiles = (M + BM - 1) / BM;
  const bool p = pdl != 0;
  if (g_persistent_min_tokens > 0 && T >= g_persistent_min_tokens && splits == 1 && !out_f32 && push == nullptr &&
      bn_override <= 0 && stages_override <= 0) {
    PersistArgs pa;
    pa.M = M;
    pa.T = T;
    pa.kb_total = a.kb_total;
    pa.w2_row_off = w2_row_off;
    pa.m_tiles = m_tiles;
    pa.tokens_fastest = a.tokens_fastest;
    pa.act = act;
    pa.ldo = ldo;
    pa.ldr = ldr;
    pa.bias = a.bias;
    pa.residual = a.residual;
    pa.out = reinterpret_cast<__nv_bfloat16*>(out);
    pa.scatter = 0;
    pa.rows_per_owner = 1;
    pa.n_peers = 0;
    pa.my_rank = 0;
    pa.seq = 0;
    pa.epoch = nullptr;
    pa.cta_counter = nullptr;
    for (int i = 0; i < 8; ++i) {
      pa.peer_out[i] = nullptr;
      pa.peer_flag[i] = nullptr;
    }
    const unsigned long long vec_addr = reinterpret_cast<unsigned long long>(out) | reinterpret_cast<unsigned long long>(bias) |
                                        reinterpret_cast<unsigned long long>(residual);
    pa.dual_rm = 0;
    if (dual && g_persistent_rowmajor && M % 16 == 0 && ldo % 8 == 0 && (vec_addr & 15ull) == 0 && bias == nullptr &&
        residual == nullptr && act == 0) {
      // SwiGLU with tokens on the TMEM lanes: one N = 256 MMA per step over [128 gate rows | 128 up rows]
      CUtensorMap ta, tb;
      rc = get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, BM, &ta);
      if (rc) return rc;
      rc = get_tensor_map(W, (unsigned long long)w_rows_total, (unsigned long long)K, (unsigned long long)ldw, 128, &tb);
      if (rc) return rc;
      pa.dual_rm = 1;
      pa.M = T;
      pa.T = 2 * M;                       // accumulator columns per full sweep: gate + up
      pa.m_tiles = (T + BM - 1) / BM;
      pa.n_tiles = (M + 127) / 128;       // 128 features (256 accumulator columns) per tile
      pa.tokens_fastest = a.tokens_fastest ? 0 : 1;
      return launch_persistent<256, false, true>(ta, tb, pa, stream, p);
    }
    if (!dual && g_persistent_rowmajor && M % 16 == 0 && ldo % 8 == 0 && (residual == nullptr || ldr % 8 == 0) &&
        (vec_addr & 15ull) == 0) {
      // tokens on the TMEM lanes: vectorised bias / residual / output rows
      pa.M = T;
      pa.T = M;
      pa.m_tiles = (T + BM - 1) / BM;
      pa.tokens_fastest = a.tokens_fastest ? 0 : 1;  // the A-row tile index is the token tile here
      // Always 256 weight rows per tile: 128-row tiles balance better over the SMs when there
      // are few tiles, but they double the operand bytes per FLOP and measured 20-45% slower
      // (1616 x 4096 -> 6144: 0.141 vs 0.097 ms).
      const int n256 = (M + 255) / 256;
      const bool narrow = false;
      CUtensorMap ta, tb;
      rc = get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, BM, &ta);
      if (rc) return rc;
      rc = get_tensor_map(W, (unsigned long long)w_rows_total, (unsigned long long)K, (unsigned long long)ldw, narrow ? 128 : 256, &tb);
      if (rc) return rc;
      pa.n_tiles = n256;
      return narrow ? launch_persistent<128, false, true>(ta, tb, pa, stream, p)
                    : launch_persistent<256, false, true>(ta, tb, pa, stream, p);
    }
    // dual: two accumulators per tile, so 128 tokens per tile keep two tiles in TMEM
    const int pbn = dual ? 128 : 256;
    pa.n_tiles = (T + pbn - 1) / pbn;
    CUtensorMap txp;
    rc = get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, (unsigned)pbn, &txp);
    if (rc) return rc;
    return dual ? launch_persistent<128, true>(tw, txp, pa, stream, p) : launch_persistent<256, false>(tw, txp, pa, stream, p);
  }
#define PRISM_GEMM_CASE(BN_)                                                                            \
  case BN_:                                                                                             \
    return dual ? launch_gemm<BN_, true>(tw, tx, a, m_tiles, splits, stages_override, stream, p)       \
                : launch_gemm<BN_, false>(tw, tx, a, m_tiles, splits, stages_override, stream, p);
  switch (bn) {
    PRISM_GEMM_CASE(16)
    PRISM_GEMM_CASE(32)
    PRISM_GEMM_CASE(64)
    PRISM_GEMM_CASE(128)
    PRISM_GEMM_CASE(256)
  }
#undef PRISM_GEMM_CASE
  return -6;
}

PRISM_API int prism_gemm_wx(const void* W, const void* X, void* out, int M, int T, int K, long long ldw, long long ldx,
                            long long ldo, int w_rows_total, const void* bias, const void* residual, long long ldr,
                            int act, int dual, int w2_row_off, int splits, int out_f32, long long split_stride,
                            int bn_override, int stages_override, void* stream_ptr, int pdl) {
  return gemm_wx_impl(W, X, out, M, T, K, ldw, ldx, ldo, w_rows_total, bias, residual, ldr, act, dual, w2_row_off, splits,
                      out_f32, split_stride, bn_override, stages_override, stream_ptr, pdl, nullptr);
}

// Fused row-parallel GEMM -> one-shot exchange: the fp32 partial of rank `my_rank`, split s,
// lands in slab (my_rank * splits + s) of every rank's buffer (peer_out[p], p < n_peers, own
// rank included; row stride ldo, slab stride split_stride, both in 8-byte elements).  Every
// element is one 8-byte word {fp32 value, low 32 bits of *epoch + point}; the consumer
// (prism_add_rmsnorm_packed) polls the words themselves, so there is no fence, counter or
// flag on this path (peer_flag and cta_counter are unused).  peer_out is a host array of
// device pointers (peer-mapped through CUDA IPC).
PRISM_API int prism_gemm_wx_push(const void* W, const void* X, int M, int T, int K, long long ldw, long long ldx,
                                 long long ldo, int w_rows_total, int splits, long long split_stride,
                                 const void* const* peer_out, const void* const* peer_flag, int n_peers, int my_rank,
                                 long long point, void* cta_counter, const void* epoch, int bn_override, int stages_override,
                                 void* stream_ptr, int pdl) {
  if (n_peers < 1 || n_peers > 8) return -20;
  PushSpec ps;
  ps.n_peers = n_peers;
  ps.my_rank = my_rank;
  ps.point = point;
  ps.push_rows = 0;
  ps.row_base = 0;
  ps.cta_counter = reinterpret_cast<int*>(cta_counter);
  ps.epoch = reinterpret_cast<const unsigned long long*>(epoch);
  for (int p = 0; p < 8; ++p) {
    ps.peer_out[p] = p < n_peers ? reinterpret_cast<float*>(const_cast<void*>(peer_out[p])) : nullptr;
    ps.peer_flag[p] = p < n_peers ? reinterpret_cast<unsigned long long*>(const_cast<void*>(peer_flag[p])) : nullptr;
  }
  return gemm_wx_impl(W, X, const_cast<void*>(peer_out[my_rank]), M, T, K, ldw, ldx, ldo, w_rows_total, nullptr, nullptr,
                      0, 0, 0, 0, splits, 1, split_stride, bn_override, stages_override, stream_ptr, pdl, &ps);
}

// Fused GEMM -> all-gather: out rows [row_base, row_base + T) = act(X W^T + bias) as bf16 are
// written into every rank's buffer (peer_out[p], row stride ldo), then flag[my_rank] on every
// rank is set to (*epoch or 0) + seq.  Used for the sharded vision tower's merger output.
PRISM_API int prism_gemm_wx_allgather(const void* W, const void* X, int M, int T, int K, long long ldw, long long ldx,
                                      long long ldo, long long row_base, const void* bias, int act,
                                      const void* const* peer_out, const void* const* peer_flag, int n_peers,
                                      int my_rank, long long seq, void* cta_counter, const void* epoch,
                                      void* stream_ptr, int pdl) {
  if (n_peers < 1 || n_peers > 8) return -20;
  PushSpec ps;
  ps.n_peers = n_peers;
  ps.my_rank = my_rank;
  ps.point = seq;
  ps.push_rows = 1;
  ps.row_base = row_base;
  ps.cta_counter = reinterpret_cast<int*>(cta_counter);
  ps.epoch = reinterpret_cast<const unsigned long long*>(epoch);
  for (int p = 0; p < 8; ++p) {
    ps.peer_out[p] = p < n_peers ? reinterpret_cast<float*>(const_cast<void*>(peer_out[p])) : nullptr;
    ps.peer_flag[p] = p < n_peers ? reinterpret_cast<unsigned long long*>(const_cast<void*>(peer_flag[p])) : nullptr;
  }
  return gemm_wx_impl(W, X, const_cast<void*>(peer_out[my_rank]), M, T, K, ldw, ldx, ldo, M, bias, nullptr, 0, act, 0, 0,
                      1, 0, 0, 0, 0, stream_ptr, pdl, &ps);
}

// Fused row-parallel GEMM -> reduce-scatter for prefill-sized steps: out rows are bf16
// X[t] . W^T (this rank's partial sum over its K shard); row t is written into the buffer of
// rank t / rows_per_owner at slab my_rank, local row t % rows_per_owner (row stride M), and
// flag[my_rank] on every rank becomes seq once all CTAs have stored.  peer_out / peer_flag:
// host arrays of device pointers (own rank included).  M a multiple of 16.  The consumer is
// prism_reduce_norm_allgather.
PRISM_API int prism_gemm_wx_scatter(const void* W, const void* X, int M, int T, int K, long long ldw, long long ldx,
                                    int rows_per_owner, const void* const* peer_out, const void* const* peer_flag,
                                    int n_peers, int my_rank, long long seq, const void* epoch, void* cta_counter,
                                    void* stream_ptr, int pdl) {
  if (T <= 0) return 0;
  if (n_peers < 1 || n_peers > 8 || rows_per_owner < 1 || (long long)rows_per_owner * n_peers < T) return -20;
  if (M % 16) return -21;
  CUtensorMap ta, tb;
  int rc = get_tensor_map(X, (unsigned long long)T, (unsigned long long)K, (unsigned long long)ldx, BM, &ta);
  if (rc) return rc;
  rc = get_tensor_map(W, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldw, 256, &tb);
  if (rc) return rc;
  PersistArgs pa;
  pa.dual_rm = 0;
  pa.M = T;
  pa.T = M;
  pa.kb_total = (K + BK - 1) / BK;
  pa.w2_row_off = 0;
  pa.m_tiles = (T + BM - 1) / BM;
  pa.n_tiles = (M + 255) / 256;
  pa.tokens_fastest = 0;
  pa.act = 0;
  pa.ldo = M;
  pa.ldr = 0;
  pa.bias = nullptr;
  pa.residual = nullptr;
  pa.out = nullptr;
  pa.scatter = 1;
  pa.rows_per_owner = rows_per_owner;
  pa.n_peers = n_peers;
  pa.my_rank = my_rank;
  pa.seq = (unsigned long long)seq;
  pa.epoch = reinterpret_cast<const unsigned long long*>(epoch);
  pa.cta_counter = reinterpret_cast<int*>(cta_counter);
  for (int i = 0; i < 8; ++i) {
    pa.peer_out[i] = i < n_peers ? reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peer_out[i])) : nullptr;
    pa.peer_flag[i] = i < n_peers ? reinterpret_cast<unsigned long long*>(const_cast<void*>(peer_flag[i])) : nullptr;
  }
  return launch_persistent<256, false, true>(ta, tb, pa, reinterpret_cast<cudaStream_t>(stream_ptr), pdl != 0);
}

PRISM_API int prism_gemm_set_persistent_rowmajor(int on) {
  g_persistent_rowmajor = on;
  return 0;
}

// Smallest token count that uses the persistent kernel (0 = never).
PRISM_API int prism_gemm_set_persistent_min_tokens(int tokens) {
  g_persistent_min_tokens = tokens;
  return 0;
}

// Shared-memory budget (bytes, 0 = whole SM) of GEMM launches with at most 32 tokens per tile.
PRISM_API int prism_gemm_set_small_tile_smem_cap(int bytes) {
  g_small_tile_smem_cap = bytes;
  return 0;
}

// Number of split-K slabs prism_gemm_wx will actually write for (K, splits).
PRISM_API int prism_gemm_effective_splits(int K, int splits) {
  const int kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  const int per = (kb_total + splits - 1) / splits;
  return (kb_total + per - 1) / per;
}

PRISM_API void prism_gemm_clear_tensor_maps() {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  g_maps.clear();
}
