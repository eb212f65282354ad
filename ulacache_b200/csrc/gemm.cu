// Weight-stationary skinny GEMM for decode:  Y[T, N] = X[T, K] * W[N, K]^T.
//
// Decode batches are small (16..512 tokens) while N is thousands wide, so the
// weight matrix takes the M side of the tcgen05 instruction (128 output
// features per CTA, always full) and the tokens take the N side (16..256, no
// padding waste).  Operands arrive by TMA (128-byte swizzle, no multicast) in a
// multi-stage mbarrier ring; one thread issues tcgen05.mma into a TMEM
// accumulator; four epilogue warps read it back with tcgen05.ld.  The ring depth
// is a launch parameter: a CTA whose K range has only a few blocks (the batched
// per-head projections) asks for that many stages, so several CTAs share an SM
// and their start-up latencies overlap.
//
// Split-K partial sums go to an fp32 scratch buffer with red.add; a second tiny
// kernel converts them.  The reference library has no GEMM of its own (it
// borrows the serving framework's), so this file has no counterpart there.
#include "ulc/launch.h"
#include "ulc/ptx.cuh"
#include "ulc/tmap.h"

namespace ulc {

constexpr int kGemmBM = 128;   // output features per CTA
constexpr int kGemmBK = 64;    // bf16 elements per stage (128 bytes)
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kGemmBM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + 4 * BN * 4 /*row maxima*/;
};

// out_mode 0: bf16 Y[T, N] plain store; 1: fp32 red.add into Y32[T, N] (split-K);
// 2: fp8 e4m3 bytes Y8 with one fp32 scale per (token, 128-feature tile) in `out_scale`
//    [T, lds] at column batch * (N / 128) + tile: the activation quantiser of the next fp8 GEMM
//    folded into this epilogue (a tile of 128 output features is exactly one quantisation group).
template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_wt_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               void* __restrict__ out, int T, int N, int K, int kb_per_split, int out_mode, int splits,
               long long ldy, long long y_bstride, int stages, int32_t* status, float* __restrict__ out_scale,
               long long lds) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * S::kStageBytes);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kGemmBM;
  const int t0 = blockIdx.y * BN;
  const int total_kb = (K + kGemmBK - 1) / kGemmBK;
  const int bz = blockIdx.z / splits;            // batch index (grid.z = batch * splits)
  const int kb_begin = (blockIdx.z % splits) * kb_per_split;
  const int kb_end = min(total_kb, kb_begin + kb_per_split);
  const int num_kb = max(0, kb_end - kb_begin);
  constexpr uint32_t kTmemCols = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    ptx::mbar_init(acc_full, 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_w);
    ptx::prefetch_tmap(&tmap_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc<kTmemCols>(tmem_holder);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_d = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (ptx::elect_one()) {
      int issued = 0;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % stages;
        const uint32_t ph = (i / stages) & 1;
        if (*abort_flag || !ptx::mbar_wait(&empty[s], ph ^ 1)) {
          if (!*abort_flag) report(status, kErrPipeline, 100 + s);
          *abort_flag = 1;
          break;
        }
        uint8_t* a = smem + s * S::kStageBytes;
        ptx::mbar_expect_tx(&full[s], S::kStageBytes);
        ptx::tma_load_3d(a, &tmap_w, &full[s], (kb_begin + i) * kGemmBK, m0, bz);
        ptx::tma_load_3d(a + S::kABytes, &tmap_x, &full[s], (kb_begin + i) * kGemmBK, t0, bz);
        issued = i + 1;
      }
      if (*abort_flag) {
        // Let copies already in flight land before the CTA gives its memory back.
        for (int i = max(0, issued - stages); i < issued; ++i)
          ptx::mbar_wait(&full[i % stages], (i / stages) & 1, 200000000LL);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc(kGemmBM, BN, 1, 1, 0, 0);
      const uint64_t smem_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem));
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % stages;
        const uint32_t ph = (i / stages) & 1;
        if (*abort_flag || !ptx::mbar_wait(&full[s], ph)) {
          if (!*abort_flag) report(status, kErrPipeline, 200 + s);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after();
        const uint64_t a_desc = ptx::umma_desc_advance(smem_desc, s * S::kStageBytes);
        const uint64_t b_desc = ptx::umma_desc_advance(a_desc, S::kABytes);
#pragma unroll
        for (int k = 0; k < kGemmBK / 16; ++k)
          ptx::umma_bf16(tmem_d, ptx::umma_desc_advance(a_desc, k * 32), ptx::umma_desc_advance(b_desc, k * 32),
                         idesc, (i | k) != 0);
        ptx::umma_commit(&empty[s]);
      }
      ptx::umma_commit(acc_full);   // fires even when num_kb == 0 or after an abort
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int q = warp & 3;                        // TMEM lane quarter this warp may read
    const bool ok = ptx::mbar_wait(acc_full, 0);
    if (!ok) {
      if (lane == 0) report(status, kErrPipeline, 300 + q);
      *abort_flag = 1;
    }
    ptx::tc_fence_after();
    const int f = m0 + q * 32 + lane;
    if (out_mode == 2) {
      // pass 1: per token the largest magnitude over this CTA's 128 features (warp, then the four warps)
      float* s_amax = reinterpret_cast<float*>(smem + stages * S::kStageBytes + 256);        // [4][BN]
      const bool live = ok && !*abort_flag && num_kb > 0;
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        if (live) { ptx::tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c, r); ptx::tmem_ld_wait(); }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t mag = (live && f < N) ? (r[j] & 0x7fffffffu) : 0u;       // |x| orders like its bit pattern
          const uint32_t m = __reduce_max_sync(0xffffffffu, mag);
          if (lane == 0) s_amax[q * BN + c + j] = __uint_as_float(m);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (live) {
#pragma unroll
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          ptx::tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c + j;
            if (t < T) {
              const float amax = fmaxf(fmaxf(s_amax[c + j], s_amax[BN + c + j]),
                                       fmaxf(s_amax[2 * BN + c + j], s_amax[3 * BN + c + j]));
              const float scale = fmaxf(amax, 1e-4f) / 448.f;
              if (f < N)
                reinterpret_cast<uint8_t*>(out)[static_cast<size_t>(bz) * y_bstride + static_cast<size_t>(t) * ldy + f] =
                    float_to_fp8_e4m3(__uint_as_float(r[j]) * (1.f / scale));
              if (q == 0 && lane == 0)
                out_scale[static_cast<size_t>(t) * lds + static_cast<size_t>(bz) * ((N + kGemmBM - 1) / kGemmBM) + blockIdx.x] = scale;
            }
          }
        }
      }
    } else if (ok && !*abort_flag && num_kb > 0) {
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        ptx::tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c, r);
        ptx::tmem_ld_wait();
        if (f < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c + j;
            if (t < T) {
              const float v = __uint_as_float(r[j]);
              const size_t o = static_cast<size_t>(bz) * y_bstride + static_cast<size_t>(t) * ldy + f;
              if (out_mode == 0) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16(v);
              else atomicAdd(reinterpret_cast<float*>(out) + o, v);
            }
          }
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc<kTmemCols>(tmem_d);
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     size_t n) {
  size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(in + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(out + i) = o;
  } else {
    for (; i < n; ++i) out[i] = __float2bfloat16(in[i]);
  }
}

template <int BN>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K,
                       int splits, int out_mode, int batch, long long ldy, long long y_bstride, int32_t* status,
                       cudaStream_t stream, float* out_scale = nullptr, long long lds = 0) {
  using S = GemmSmem<BN>;
  static PerDeviceOnce once;
  const int attr_rc = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_wt_kernel<BN>), S::kBytes, once);
  if (attr_rc != 0) return attr_rc;
  const int total_kb = (K + kGemmBK - 1) / kGemmBK;
  const int kb_per_split = (total_kb + splits - 1) / splits;
  dim3 grid((N + kGemmBM - 1) / kGemmBM, (T + BN - 1) / BN, splits * batch);
  // no deeper a ring than the K blocks one CTA walks: the shared memory saved lets CTAs share an SM
  const int stages = kb_per_split < 2 ? 2 : (kb_per_split < S::kStages ? kb_per_split : S::kStages);
  const size_t smem_bytes = static_cast<size_t>(stages) * S::kStageBytes + 1024 /*align*/ + 256 /*barriers*/ +
                            (out_mode == 2 ? 4 * BN * sizeof(float) : 0);
  gemm_wt_kernel<BN><<<grid, kGemmThreads, smem_bytes, stream>>>(tw, tx, out, T, N, K, kb_per_split,
                                                                  out_mode, splits, ldy, y_bstride, stages, status,
                                                                  out_scale, lds);
  return static_cast<int>(cudaGetLastError());
}

// [batch][rows][cols] bf16 tensor with element strides (row pitch ld, batch pitch bstride).
static int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t batch,
                             uint64_t ld, uint64_t bstride, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 7) || (bstride & 7)) return -kErrAlignment;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, (batch > 1 ? bstride : rows * ld) * 2};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kGemmBK), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace ulc

extern "C" {

// Batched form: for every b < batch,  Y_b[T,N] = X_b[T,K] * W_b[N,K]^T  with element strides
// (ldx, x_bstride), (ldw, w_bstride), (ldy, y_bstride); all bf16.  splits > 1 (batch == 1 only)
// needs `scratch_f32` of T*N floats.  K and every stride must be multiples of 8.
int ulc_gemm_wt_bf16_batched(const void* x, const void* w, void* y, int T, int N, int K, long long ldx,
                             long long ldw, long long ldy, int batch, long long x_bstride, long long w_bstride,
                             long long y_bstride, int splits, void* scratch_f32, int32_t* status,
                             cudaStream_t stream) {
  using namespace ulc;
  if (T <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -kErrAlignment;
  if (splits < 1) splits = 1;
  if (splits > 1 && (scratch_f32 == nullptr || batch != 1)) return -kErrUnsupported;
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
  CUtensorMap tw, tx;
  int r = make_tmap_3d_bf16(&tw, w, N, K, batch, ldw, w_bstride, kGemmBM);
  if (r != 0) return r;
  r = make_tmap_3d_bf16(&tx, x, T, K, batch, ldx, x_bstride, bn);
  if (r != 0) return r;
  void* out = y;
  int mode = 0;
  long long oy = ldy, ob = y_bstride;
  if (splits > 1) {
    cudaMemsetAsync(scratch_f32, 0, sizeof(float) * static_cast<size_t>(T) * N, stream);
    out = scratch_f32;
    mode = 1;
    oy = N;
    ob = 0;
  }
  switch (bn) {
    case 16: r = launch_gemm<16>(tw, tx, out, T, N, K, splits, mode, batch, oy, ob, status, stream); break;
    case 32: r = launch_gemm<32>(tw, tx, out, T, N, K, splits, mode, batch, oy, ob, status, stream); break;
    case 64: r = launch_gemm<64>(tw, tx, out, T, N, K, splits, mode, batch, oy, ob, status, stream); break;
    default: r = launch_gemm<128>(tw, tx, out, T, N, K, splits, mode, batch, oy, ob, status, stream); break;
  }
  if (r != 0) return r;
  if (splits > 1) {
    const size_t n = static_cast<size_t>(T) * N;
    const int blocks = static_cast<int>((n / 4 + 255) / 256) + 1;
    // the conversion assumes a dense [T, N] result
    if (ldy != N) return -kErrUnsupported;
    cast_f32_bf16_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(scratch_f32),
                                                     reinterpret_cast<__nv_bfloat16*>(y), n);
    r = static_cast<int>(cudaGetLastError());
  }
  return r;
}

// Batched GEMM whose result is quantised in the epilogue: for every b < batch,
// Y8_b[T, N] = fp8(X_b W_b^T) with one fp32 scale per (token, 128 features), stored at
// y8[t * ldy + b * y_bstride + n] (bytes) and scales[t * lds + b * ceil(N / 128) + n / 128].
int ulc_gemm_wt_bf16_batched_quant(const void* x, const void* w, void* y8, float* scales, int T, int N, int K,
                                   long long ldx, long long ldw, long long ldy, long long lds, int batch,
                                   long long x_bstride, long long w_bstride, long long y_bstride, int32_t* status,
                                   cudaStream_t stream) {
  using namespace ulc;
  if (T <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -kErrAlignment;
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
  CUtensorMap tw, tx;
  int r = make_tmap_3d_bf16(&tw, w, N, K, batch, ldw, w_bstride, kGemmBM);
  if (r != 0) return r;
  r = make_tmap_3d_bf16(&tx, x, T, K, batch, ldx, x_bstride, bn);
  if (r != 0) return r;
  switch (bn) {
    case 16: return launch_gemm<16>(tw, tx, y8, T, N, K, 1, 2, batch, ldy, y_bstride, status, stream, scales, lds);
    case 32: return launch_gemm<32>(tw, tx, y8, T, N, K, 1, 2, batch, ldy, y_bstride, status, stream, scales, lds);
    case 64: return launch_gemm<64>(tw, tx, y8, T, N, K, 1, 2, batch, ldy, y_bstride, status, stream, scales, lds);
    default: return launch_gemm<128>(tw, tx, y8, T, N, K, 1, 2, batch, ldy, y_bstride, status, stream, scales, lds);
  }
}

// Y[T,N] (bf16) = X[T,K] (bf16, row pitch ldx elements) * W[N,K]^T (bf16, row pitch ldw).
// splits > 1 requires `scratch_f32` of T*N floats; it is cleared here, accumulated
// with red.add and converted to bf16 at the end.  K, ldx and ldw must be multiples of 8.
int ulc_gemm_wt_bf16(const void* x, const void* w, void* y, int T, int N, int K, int ldx, int ldw,
                     int splits, void* scratch_f32, int32_t* status, cudaStream_t stream) {
  return ulc_gemm_wt_bf16_batched(x, w, y, T, N, K, ldx, ldw, N, 1, 0, 0, 0, splits, scratch_f32, status, stream);
}

}  // extern "C"
