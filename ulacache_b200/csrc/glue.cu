// Fused element-wise stages of the decode layer.  Each kernel replaces a chain of
// six to ten framework element-wise launches, which at decode batch sizes cost
// more in launch gaps than in work.
//
//   add_rmsnorm_quant : x += delta; h = rmsnorm(x) * w; fp8 quantise h per 128 columns
//   mla_prep          : split the fused input projection: rmsnorm + fp8 quant of the q
//                       latent, rmsnorm of the KV latent, rotary on the shared key part
//   q_prep            : rotary on every head's q_rope (written into the attention query
//                       layout), rotary + fp8 quant of the indexer queries with the
//                       quantisation scale folded into the indexer head weights
//   moe_route / moe_gather / moe_combine : sigmoid top-k routing with a counting sort
//                       by expert, the row gather for the grouped GEMM, and the weighted
//                       un-permute fused with the shared expert and the residual
//
// The reference library has no model code; these stages belong to the serving
// framework it patches.
#include "ulc/ptx.cuh"

namespace ulc {

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// One CTA (1024 threads) per row; every thread owns 8 consecutive columns, so the row and all the
// partial results added to it are in flight at once as independent 16-byte loads (a decode batch
// gives this kernel only a few dozen CTAs, and its time is the latency of those loads).
// H is a multiple of 128 and at most 8192.
// x (bf16, in/out when delta != null): x += delta.  h_out (nullable): normed bf16.
// q/s (nullable): fp8 + one scale per 128 columns of the normed row.
constexpr int kNormThreads = 1024;
constexpr int kNormMaxSlots = 8;

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = __bfloat1622float2(p2[j]);
    f[2 * j] = a.x;
    f[2 * j + 1] = a.y;
  }
}

__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_quant_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                         const float* __restrict__ delta32, int n_slots, long long slot_stride,
                         const __nv_bfloat16* __restrict__ w, float eps, int H,
                         __nv_bfloat16* __restrict__ h_out, uint8_t* __restrict__ q, float* __restrict__ s) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const int t = threadIdx.x;
  const int c = t * 8;
  const bool active = c < H;
  __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
  float ss = 0.f;
  uint4 wraw = make_uint4(0, 0, 0, 0);
  if (active) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
    wraw = *reinterpret_cast<const uint4*>(w + c);
    // `delta` may be n_slots partial results (one per rank, slot_stride elements apart): the reduce
    // phase of the one-shot all-reduce happens here, in fp32.  All slots are loaded before any is used.
    uint4 dr[kNormMaxSlots];
    if (delta) {
#pragma unroll
      for (int sl = 0; sl < kNormMaxSlots; ++sl)
        if (sl < n_slots)
          dr[sl] = *reinterpret_cast<const uint4*>(delta + sl * slot_stride + static_cast<size_t>(row) * H + c);
    }
    float4 d4a = make_float4(0.f, 0.f, 0.f, 0.f), d4b = d4a;
    if (delta32) {
      d4a = *reinterpret_cast<const float4*>(delta32 + static_cast<size_t>(row) * H + c);
      d4b = *reinterpret_cast<const float4*>(delta32 + static_cast<size_t>(row) * H + c + 4);
    }
    unpack8(raw, v);
    if (delta) {
#pragma unroll
      for (int sl = 0; sl < kNormMaxSlots; ++sl) {
        if (sl < n_slots) {
          float d[8];
          unpack8(dr[sl], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += d[j];
        }
      }
    }
    if (delta32) {
      v[0] += d4a.x; v[1] += d4a.y; v[2] += d4a.z; v[3] += d4a.w;
      v[4] += d4b.x; v[5] += d4b.y; v[6] += d4b.z; v[7] += d4b.w;
    }
    if (delta || delta32) {
      // the residual stream is kept in bf16: round once and norm what was stored
      uint4 ow;
      uint32_t* o32 = reinterpret_cast<uint32_t*>(&ow);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 o = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        o32[j] = *reinterpret_cast<uint32_t*>(&o);
        const float2 r = __bfloat1622float2(o);
        v[2 * j] = r.x;
        v[2 * j + 1] = r.y;
      }
      *reinterpret_cast<uint4*>(xr + c) = ow;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / H + eps);
  // Inactive lanes take part in the shuffles below with zeros (H is a multiple of 128 columns =
  // 16 threads, so a 16-lane group is either entirely active or entirely inactive).
  float wv[8];
  unpack8(wraw, wv);
  float y[8];
  uint4 ow;
  uint32_t* o32 = reinterpret_cast<uint32_t*>(&ow);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // the reference path rounds the normed activation to bf16 before quantising
    __nv_bfloat162 o = __floats2bfloat162_rn(v[2 * j] * rstd * wv[2 * j], v[2 * j + 1] * rstd * wv[2 * j + 1]);
    o32[j] = *reinterpret_cast<uint32_t*>(&o);
    const float2 r = __bfloat1622float2(o);
    y[2 * j] = r.x;
    y[2 * j + 1] = r.y;
    amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
  }
  if (active && h_out) *reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * H + c) = ow;
  if (q) {
    // 128 columns = 16 consecutive threads
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-4f) / 448.f;
    const float inv = 1.f / scale;
    uint2 pk = make_uint2(0, 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      pk.x |= static_cast<uint32_t>(float_to_fp8_e4m3(y[k] * inv)) << (8 * k);
      pk.y |= static_cast<uint32_t>(float_to_fp8_e4m3(y[4 + k] * inv)) << (8 * k);
    }
    if (active) {
      *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * H + c) = pk;
      if ((t & 15) == 0) s[static_cast<size_t>(row) * (H / 128) + c / 128] = scale;
    }
  }
}


// One CTA (256 threads) per token.  `fused` row = [ q latent (q_lora) | kv latent (512) | k rope (64) | ... ].
//   q8/qs     : fp8 + scales of rmsnorm(q latent) * q_norm
//   latent    : bf16 rmsnorm(kv latent) * kv_norm               [B, 512]
//   k_rope    : bf16 rotary(k rope) at position lengths[b]      [B, 64]   (pairs (i, i + 32))
__global__ void __launch_bounds__(256)
mla_prep_kernel(const __nv_bfloat16* __restrict__ fused, long long ld, int q_lora,
                const __nv_bfloat16* __restrict__ q_norm, const __nv_bfloat16* __restrict__ kv_norm, float eps,
                const float* __restrict__ cos_sin, const int32_t* __restrict__ lengths,
                uint8_t* __restrict__ q8, float* __restrict__ qs, __nv_bfloat16* __restrict__ latent,
                __nv_bfloat16* __restrict__ k_rope) {
  __shared__ float scratch[32];
  const int b = blockIdx.x, t = threadIdx.x;
  const __nv_bfloat16* row = fused + static_cast<size_t>(b) * ld;
  // ---- q latent: up to 2048 columns, 4 per thread per pass
  float v[2][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c = (i * 256 + t) * 4;
    if (c < q_lora) {
      const uint2 raw = *reinterpret_cast<const uint2*>(row + c);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(p2[0]), bb = __bfloat1622float2(p2[1]);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = bb.x; v[i][3] = bb.y;
#pragma unroll
      for (int k = 0; k < 4; ++k) ss += v[i][k] * v[i][k];
    }
  }
  const float rstd = rsqrtf(block_sum(ss, scratch) / q_lora + eps);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c = (i * 256 + t) * 4;
    if (c < q_lora) {
      float y[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        y[k] = __bfloat162float(__float2bfloat16(v[i][k] * rstd * __bfloat162float(q_norm[c + k])));
      float amax = fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3])));
      amax = warp_max(amax);
      const float scale = fmaxf(amax, 1e-4f) / 448.f;
      const float inv = 1.f / scale;
      uint32_t pk = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) pk |= static_cast<uint32_t>(float_to_fp8_e4m3(y[k] * inv)) << (8 * k);
      *reinterpret_cast<uint32_t*>(q8 + static_cast<size_t>(b) * q_lora + c) = pk;
      if ((t & 31) == 0) qs[static_cast<size_t>(b) * (q_lora / 128) + c / 128] = scale;
    }
  }
  // ---- kv latent: 512 columns on threads 0..127
  float u[4] = {0.f, 0.f, 0.f, 0.f};
  float s2 = 0.f;
  if (t < 128) {
    const uint2 raw = *reinterpret_cast<const uint2*>(row + q_lora + t * 4);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(p2[0]), bb = __bfloat1622float2(p2[1]);
    u[0] = a.x; u[1] = a.y; u[2] = bb.x; u[3] = bb.y;
    s2 = u[0] * u[0] + u[1] * u[1] + u[2] * u[2] + u[3] * u[3];
  }
  const float rstd2 = rsqrtf(block_sum(s2, scratch) / 512.f + eps);
  if (t < 128) {
    __nv_bfloat162 o0 = __floats2bfloat162_rn(u[0] * rstd2 * __bfloat162float(kv_norm[t * 4]),
                                              u[1] * rstd2 * __bfloat162float(kv_norm[t * 4 + 1]));
    __nv_bfloat162 o1 = __floats2bfloat162_rn(u[2] * rstd2 * __bfloat162float(kv_norm[t * 4 + 2]),
                                              u[3] * rstd2 * __bfloat162float(kv_norm[t * 4 + 3]));
    uint2 ow;
    ow.x = *reinterpret_cast<uint32_t*>(&o0);
    ow.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(latent + static_cast<size_t>(b) * 512 + t * 4) = ow;
  } else if (t < 160) {
    // ---- rotary on the 64-wide shared key part: thread handles the pair (i, i + 32)
    const int i = t - 128;
    const float* cs = cos_sin + static_cast<size_t>(lengths[b]) * 64;
    const float c = cs[i], sn = cs[32 + i];
    const float a = __bfloat162float(row[q_lora + 512 + i]), bb = __bfloat162float(row[q_lora + 512 + 32 + i]);
    k_rope[static_cast<size_t>(b) * 64 + i] = __float2bfloat16(a * c - bb * sn);
    k_rope[static_cast<size_t>(b) * 64 + 32 + i] = __float2bfloat16(bb * c + a * sn);
  }
}

// Grid (B, 2), 256 threads.  `qb` row = [ heads x (nope 128 | rope 64) | 64 indexer heads x 128 ].
//  y == 0: q_nope -> q_nope_t [heads, B, 128] (ready for the batched absorb GEMM),
//          rotary(q_rope) -> q_rope_out [B, heads, 64]
//  y == 1: indexer queries: rotary on the first 64 dims of each head, fp8 quantise per head,
//          iw_out[b, h] = iw[b, h] * scale * head_scale      (iw read from `fused` at iw_off)
__global__ void __launch_bounds__(256)
q_prep_kernel(const __nv_bfloat16* __restrict__ qb, long long ld, int heads, int B,
              const float* __restrict__ cos_sin, const int32_t* __restrict__ lengths,
              __nv_bfloat16* __restrict__ q_nope_t, __nv_bfloat16* __restrict__ q_rope_out,
              const __nv_bfloat16* __restrict__ fused, long long fused_ld, int iw_off, float head_scale,
              uint8_t* __restrict__ iq8, float* __restrict__ iw_out) {
  const int b = blockIdx.x, t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const __nv_bfloat16* row = qb + static_cast<size_t>(b) * ld;
  const float* cs = cos_sin + static_cast<size_t>(lengths[b]) * 64;
  if (blockIdx.y == 0) {
    // one warp per head: 128 nope values (4 per lane) + 64 rope values (pair per lane)
    for (int h = warp; h < heads; h += 8) {
      const __nv_bfloat16* src = row + h * 192;
      if (q_nope_t)
        *reinterpret_cast<uint2*>(q_nope_t + (static_cast<size_t>(h) * B + b) * 128 + lane * 4) =
            *reinterpret_cast<const uint2*>(src + lane * 4);
      const float c = cs[lane], sn = cs[32 + lane];
      const float a = __bfloat162float(src[128 + lane]), bb = __bfloat162float(src[128 + 32 + lane]);
      __nv_bfloat16* dst = q_rope_out + (static_cast<size_t>(b) * heads + h) * 64;
      dst[lane] = __float2bfloat16(a * c - bb * sn);
      dst[32 + lane] = __float2bfloat16(bb * c + a * sn);
    }
  } else {
    const __nv_bfloat16* iq = row + heads * 192;
    for (int h = warp; h < 64; h += 8) {
      const __nv_bfloat16* src = iq + h * 128;
      // lane owns dims {lane, lane + 32, lane + 64, lane + 96}: the rotary pair is in-lane
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(src[lane + 32 * i]);
      const float c = cs[lane], sn = cs[32 + lane];
      const float a = x[0], bb = x[1];
      x[0] = __bfloat162float(__float2bfloat16(a * c - bb * sn));
      x[1] = __bfloat162float(__float2bfloat16(bb * c + a * sn));
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
      amax = warp_max(amax);
      const float scale = fmaxf(amax, 1e-4f) / 448.f;
      const float inv = 1.f / scale;
      uint8_t* dst = iq8 + (static_cast<size_t>(b) * 64 + h) * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = float_to_fp8_e4m3(x[i] * inv);
      if (lane == 0)
        iw_out[static_cast<size_t>(b) * 64 + h] =
            __bfloat162float(fused[static_cast<size_t>(b) * fused_ld + iw_off + h]) * head_scale * scale;
    }
  }
}


// Sigmoid top-k routing (E <= 256 experts, topk <= 8, any B):
//   logits [B, E] bf16 (router GEMM output), bias [E] fp32 (added for selection only)
//   choice [B, topk]     : selected experts, best first (ties go to the lower expert index)
//   gate [B, topk]       : sigmoid score of each choice, normalised over the choices, times routed_scale
// Order-preserving map of a float onto uint32 (NaN sorts lowest, with -inf); 0 is never produced.
__device__ __forceinline__ uint32_t route_key(float x) {
  uint32_t u = __float_as_uint(x);
  if (x != x) u = 0xff800000u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One warp per token; lane l owns experts l, l + 32, ...  Each round takes the warp maximum of the
// lanes' best remaining keys with one redux instruction and resolves ties to the lowest expert
// index with a second one; only the owning lane rescans its (at most 8) experts.
__global__ void __launch_bounds__(256)
moe_topk_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ bias, int B, int E, int topk,
                float routed_scale, float* __restrict__ gate, int32_t* __restrict__ choice) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * 8 + warp;          // one warp per token
  if (b >= B) return;
  const int per = (E + 31) / 32;                // experts per lane, <= 8
  float sc[8];
  uint32_t key[8];                              // 0: taken or absent
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + 32 * j;
    if (j < per && e < E) {
      const float z = __bfloat162float(logits[static_cast<size_t>(b) * E + e]);
      sc[j] = 1.f / (1.f + __expf(-z));
      key[j] = route_key(sc[j] + (bias ? bias[e] : 0.f));
    } else {
      sc[j] = 0.f;
      key[j] = 0u;
    }
  }
  uint32_t best = 0u;
  int best_j = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) if (key[j] > best) { best = key[j]; best_j = j; }   // ties: lower expert
  float myg = 0.f, gsum = 0.f;
  int mye = 0;
  // fully unrolled: a run-time trip count would put per-round state in local memory
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k >= topk) continue;
    const uint32_t top = __reduce_max_sync(0xffffffffu, best);
    const uint32_t be = __reduce_min_sync(0xffffffffu, best == top ? static_cast<uint32_t>(lane + 32 * best_j) : 0xffffffffu);
    const int owner_lane = be & 31, owner_j = be >> 5;
    float val = 0.f;
    if (lane == owner_lane) {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (j == owner_j) { val = sc[j]; key[j] = 0u; }
      best = 0u;
      best_j = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) if (key[j] > best) { best = key[j]; best_j = j; }
    }
    val = __shfl_sync(0xffffffffu, val, owner_lane);
    gsum += val;
    if (lane == k) { myg = val; mye = static_cast<int>(be); }
  }
  if (lane < topk) {
    gate[static_cast<size_t>(b) * topk + lane] = myg / fmaxf(gsum, 1e-20f) * routed_scale;
    choice[static_cast<size_t>(b) * topk + lane] = mye;
  }
}

// Where to put the shared expert in the list of experts the grouped GEMM walks.  The GEMM deals
// items (expert, feature tile) round robin to `grid` persistent CTAs, `tiles` items per expert, and
// the shared expert's items take about twice as long (its rows need a second pass).  With
// n_items % grid != 0 the first CTAs get one item more; the shared expert goes to the first list
// position whose items all fall on CTAs without that extra item.  tiles <= 0 or no such position:
// last (ascending expert order, the default).
__host__ __device__ inline int shared_expert_position(int n_routed, int tiles, int grid) {
  if (tiles <= 0 || grid <= 0 || tiles > grid) return n_routed;
  const long long n_items = static_cast<long long>(n_routed + 1) * tiles;
  const int rem = static_cast<int>(n_items % grid);
  if (rem == 0) return n_routed;
  for (int p = 0; p <= n_routed; ++p) {
    const int start = static_cast<int>((static_cast<long long>(p) * tiles) % grid);
    if (start >= rem && start + tiles <= grid) return p;
  }
  return n_routed;
}

// Counting sort of the (token, choice) pairs by local expert.  With shared_n >= 0 an extra
// expert `n_local` (the shared expert) receives tokens shared_lo .. shared_lo + shared_n - 1,
// one row each, after the routed rows: offs then has n_local + 2 entries.
// PLACED = false is the plain form (ascending list, shared expert last); the placement rule, its
// extra barrier and the second list exist only in the PLACED = true instantiation.
template <bool PLACED>
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int32_t* __restrict__ choice, int B, int topk, int lo, int n_local, int shared_lo,
                int shared_n, int32_t* __restrict__ offs, int32_t* __restrict__ slot_token,
                int32_t* __restrict__ inv_slot, int32_t* __restrict__ active, int32_t* __restrict__ active2,
                int tiles_a, int tiles_b, int grid) {
  __shared__ int s_count[257];
  __shared__ int s_cursor[257];
  __shared__ int s_warp_rows[8], s_warp_active[8];
  __shared__ int s_place[2];      // position of the shared expert in `active` and `active2`
  const int t = threadIdx.x;
  for (int i = t; i <= 256; i += 1024) { s_count[i] = 0; s_cursor[i] = 0; }
  __syncthreads();
  for (int i = t; i < B * topk; i += 1024) {
    const int le = choice[i] - lo;
    if (le >= 0 && le < n_local) atomicAdd(&s_count[le], 1);
  }
  __syncthreads();
  // Exclusive scan of the per-expert row counts and, with the same ballots, the ascending list
  // of experts that received rows (for the grouped GEMM): thread e < 256 owns expert e.
  int c = 0, incl = 0;
  uint32_t has_rows = 0;
  if (t < 256) {
    c = t < n_local ? s_count[t] : 0;
    incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if ((t & 31) >= o) incl += v;
    }
    has_rows = __ballot_sync(0xffffffffu, c > 0);
    if ((t & 31) == 31) { s_warp_rows[t >> 5] = incl; s_warp_active[t >> 5] = __popc(has_rows); }
  }
  __syncthreads();
  if constexpr (PLACED) {
    if (t == 0) {
      int n_routed = 0;
      for (int w = 0; w < 8; ++w) n_routed += s_warp_active[w];
      s_place[0] = shared_expert_position(n_routed, tiles_a, grid);
      s_place[1] = shared_expert_position(n_routed, tiles_b, grid);
    }
    __syncthreads();
  }
  if (t < 256) {
    int row_base = 0, act_base = 0;
    for (int w = 0; w < (t >> 5); ++w) { row_base += s_warp_rows[w]; act_base += s_warp_active[w]; }
    const int excl = row_base + incl - c;
    const bool with_shared = shared_n > 0;
    if (t < n_local) {
      s_count[t] = excl;
      offs[t] = excl;
      if (c > 0) {
        // rank among the routed experts that received rows; the shared expert is inserted at s_place
        const int r = act_base + __popc(has_rows & ((1u << (t & 31)) - 1u));
        if constexpr (PLACED) {
          if (active != nullptr) active[1 + r + ((with_shared && r >= s_place[0]) ? 1 : 0)] = t;
          if (active2 != nullptr) active2[1 + r + ((with_shared && r >= s_place[1]) ? 1 : 0)] = t;
        } else {
          if (active != nullptr) active[1 + r] = t;
        }
      }
    }
    if (t == 255) {
      const int total = row_base + incl, n_active = act_base + __popc(has_rows);
      offs[n_local] = total;
      s_count[n_local] = total;
      if (shared_n >= 0) offs[n_local + 1] = total + shared_n;
      if (active != nullptr) {
        if (with_shared) active[1 + (PLACED ? s_place[0] : n_active)] = n_local;
        active[0] = n_active + (with_shared ? 1 : 0);
      }
      if constexpr (PLACED) {
        if (active2 != nullptr) {
          if (with_shared) active2[1 + s_place[1]] = n_local;
          active2[0] = n_active + (with_shared ? 1 : 0);
        }
      }
    }
  }
  __syncthreads();
  for (int i = t; i < B * topk; i += 1024) {
    const int le = choice[i] - lo;
    int slot = -1;
    if (le >= 0 && le < n_local) {
      slot = s_count[le] + atomicAdd(&s_cursor[le], 1);
      slot_token[slot] = i / topk;
    }
    inv_slot[i] = slot;
  }
  for (int i = t; i < shared_n; i += 1024) slot_token[s_count[n_local] + i] = shared_lo + i;
}

// Rows of the grouped GEMM input: x8p[slot] = x8[token(slot)], sxp likewise.  One warp per slot.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint8_t* __restrict__ x8, const float* __restrict__ sx, const int32_t* __restrict__ slot_token,
                  const int32_t* __restrict__ offs, int n_local, int K, uint8_t* __restrict__ x8p,
                  float* __restrict__ sxp, int max_slots) {
  const int total = offs[n_local];
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; slot < total && slot < max_slots; slot += warps) {
    const int tok = slot_token[slot];
    const uint4* src = reinterpret_cast<const uint4*>(x8 + static_cast<size_t>(tok) * K);
    uint4* dst = reinterpret_cast<uint4*>(x8p + static_cast<size_t>(slot) * K);
    for (int c = lane; c < K / 16; c += 32) dst[c] = src[c];
    const int KB = K / 128;
    for (int c = lane; c < KB; c += 32) sxp[static_cast<size_t>(slot) * KB + c] = sx[static_cast<size_t>(tok) * KB + c];
  }
}

// out[b] = sum_k gate[b,k] * y[inv_slot[b,k]] + shared[b]   (bf16 out, fp32 accumulation).
// The result is also stored to every buffer of `peers` (scatter phase of a one-shot all-reduce).
struct PeerOut { void* p[8]; int n; };

__global__ void __launch_bounds__(512)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ inv_slot,
                   const float* __restrict__ gate, const __nv_bfloat16* __restrict__ shared, int topk, int H,
                   __nv_bfloat16* __restrict__ out, PeerOut peers, int rows_per_peer,
                   const int32_t* __restrict__ shared_slot0, int shared_lo, int shared_n) {
  const int b = blockIdx.x;
  // the shared expert's output for tokens shared_lo .. shared_lo + shared_n - 1 may sit in y
  // itself, from row *shared_slot0 on (it ran as one more expert of the grouped GEMM)
  const __nv_bfloat16* srow = shared ? shared + static_cast<size_t>(b) * H : nullptr;
  if (shared_slot0 != nullptr)
    srow = (b >= shared_lo && b < shared_lo + shared_n)
               ? y + (static_cast<size_t>(*shared_slot0) + (b - shared_lo)) * H : nullptr;
  // all-reduce scatter: row b goes to row b of every peer; reduce-scatter: row b belongs to
  // peer b / rows_per_peer and lands at its row b % rows_per_peer
  const int first = rows_per_peer > 0 ? b / rows_per_peer : 0;
  const int last = rows_per_peer > 0 ? first + 1 : peers.n;
  const int drow = rows_per_peer > 0 ? b % rows_per_peer : b;
  int sl[8];
  float g[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    sl[k] = k < topk ? inv_slot[static_cast<size_t>(b) * topk + k] : -1;
    g[k] = k < topk ? gate[static_cast<size_t>(b) * topk + k] : 0.f;
  }
  // 8 columns (16 bytes) per thread and step; every selected row's load is issued before use
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 raw[9];
    if (srow) raw[8] = *reinterpret_cast<const uint4*>(srow + c);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (sl[k] >= 0) raw[k] = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(sl[k]) * H + c);
    if (srow) unpack8(raw[8], acc);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (sl[k] >= 0) {
        float f[8];
        unpack8(raw[k], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(g[k], f[j], acc[j]);
      }
    }
    uint4 ow;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&ow);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 o = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      o32[j] = *reinterpret_cast<uint32_t*>(&o);
    }
    if (out) *reinterpret_cast<uint4*>(out + static_cast<size_t>(b) * H + c) = ow;
    for (int r = first; r < last && r < peers.n; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peers.p[r]) + static_cast<size_t>(drow) * H + c) = ow;
  }
  if (peers.n > 0) ptx::cta_release_peer_stores();
}

// Copies up to four local segments to the same offsets of every peer's buffer (the send half
// of an all-gather through peer memory).  blockIdx.y = peer; 16-byte units.
struct PutSegs { const uint4* src[4]; long long dst_off[4]; long long units[4]; int n; };

__global__ void __launch_bounds__(256)
peer_put_kernel(PutSegs segs, PeerOut peers) {
  uint8_t* base = reinterpret_cast<uint8_t*>(peers.p[blockIdx.y]);
  for (int sg = 0; sg < segs.n; ++sg) {
    uint4* dst = reinterpret_cast<uint4*>(base + segs.dst_off[sg]);
    const uint4* src = segs.src[sg];
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < segs.units[sg];
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      dst[i] = src[i];
  }
  ptx::cta_release_peer_stores();
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// delta (bf16) may hold n_slots partial tensors slot_stride elements apart (summed in fp32);
// pass n_slots = 1 for a plain residual add.
int ulc_add_rmsnorm_quant(void* x, const void* delta, const float* delta32, int n_slots, long long slot_stride,
                          const void* w, float eps, int rows, int H, void* h_out, void* q, float* s,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H % 128) || H > 8192 || n_slots < 1 || n_slots > kNormMaxSlots || (slot_stride % 8)) return -kErrUnsupported;
  add_rmsnorm_quant_kernel<<<rows, kNormThreads, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(delta), delta32, n_slots, slot_stride,
      reinterpret_cast<const __nv_bfloat16*>(w), eps, H, reinterpret_cast<__nv_bfloat16*>(h_out),
      reinterpret_cast<uint8_t*>(q), s);
  return static_cast<int>(cudaGetLastError());
}

int ulc_mla_prep(const void* fused, long long ld, int q_lora, const void* q_norm, const void* kv_norm, float eps,
                 const float* cos_sin, const int32_t* lengths, int B, void* q8, float* qs, void* latent,
                 void* k_rope, cudaStream_t stream) {
  if (B <= 0) return 0;
  if ((q_lora % 128) || q_lora > 2048 || (ld % 4)) return -kErrUnsupported;
  mla_prep_kernel<<<B, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(fused), ld, q_lora, reinterpret_cast<const __nv_bfloat16*>(q_norm),
      reinterpret_cast<const __nv_bfloat16*>(kv_norm), eps, cos_sin, lengths, reinterpret_cast<uint8_t*>(q8), qs,
      reinterpret_cast<__nv_bfloat16*>(latent), reinterpret_cast<__nv_bfloat16*>(k_rope));
  return static_cast<int>(cudaGetLastError());
}

int ulc_q_prep(const void* qb, long long ld, int heads, int B, const float* cos_sin, const int32_t* lengths,
               void* q_nope_t, void* q_rope, const void* fused, long long fused_ld, int iw_off, float head_scale,
               void* iq8, float* iw_out, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (ld % 4) return -kErrUnsupported;
  q_prep_kernel<<<dim3(B, 2), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(qb), ld, heads, B, cos_sin, lengths,
      reinterpret_cast<__nv_bfloat16*>(q_nope_t), reinterpret_cast<__nv_bfloat16*>(q_rope),
      reinterpret_cast<const __nv_bfloat16*>(fused), fused_ld, iw_off, head_scale,
      reinterpret_cast<uint8_t*>(iq8), iw_out);
  return static_cast<int>(cudaGetLastError());
}

int ulc_moe_topk(const void* logits, const float* bias, int B, int E, int topk, float routed_scale, float* gate,
                 int32_t* choice, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (E > 256 || topk > 8) return -kErrUnsupported;
  moe_topk_kernel<<<(B + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), bias, B, E, topk,
                                                   routed_scale, gate, choice);
  return static_cast<int>(cudaGetLastError());
}

// active / active2 (nullable): [count, expert ids] lists for two grouped GEMMs with tiles_a / tiles_b
// feature tiles per expert on `grid` persistent CTAs (see shared_expert_position; 0 tiles = plain
// ascending order with the shared expert last).
int ulc_moe_sort_ex(const int32_t* choice, int B, int topk, int lo, int n_local, int shared_lo, int shared_n,
                    int32_t* offs, int32_t* slot_token, int32_t* inv_slot, int32_t* active, int32_t* active2,
                    int tiles_a, int tiles_b, int grid, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (topk > 8 || n_local > 256 || shared_n < -1 || shared_lo < 0 || shared_lo + shared_n > B) return -kErrUnsupported;
  if (tiles_a > 0 || tiles_b > 0 || active2 != nullptr)
    moe_sort_kernel<true><<<1, 1024, 0, stream>>>(choice, B, topk, lo, n_local, shared_lo, shared_n, offs, slot_token,
                                                  inv_slot, active, active2, tiles_a, tiles_b, grid);
  else
    moe_sort_kernel<false><<<1, 1024, 0, stream>>>(choice, B, topk, lo, n_local, shared_lo, shared_n, offs, slot_token,
                                                   inv_slot, active, nullptr, 0, 0, 0);
  return static_cast<int>(cudaGetLastError());
}

int ulc_moe_sort(const int32_t* choice, int B, int topk, int lo, int n_local, int shared_lo, int shared_n,
                 int32_t* offs, int32_t* slot_token, int32_t* inv_slot, int32_t* active, cudaStream_t stream) {
  return ulc_moe_sort_ex(choice, B, topk, lo, n_local, shared_lo, shared_n, offs, slot_token, inv_slot, active, nullptr,
                         0, 0, 0, stream);
}

// Host copy of the placement rule, for tests.
int ulc_shared_expert_position(int n_routed, int tiles, int grid) { return shared_expert_position(n_routed, tiles, grid); }

int ulc_moe_gather(const void* x8, const float* sx, const int32_t* slot_token, const int32_t* offs, int n_local,
                   int K, void* x8p, float* sxp, int max_slots, cudaStream_t stream) {
  if (max_slots <= 0) return 0;
  if (K % 128) return -kErrUnsupported;
  int blocks = (max_slots + 7) / 8;
  if (blocks > 592) blocks = 592;
  moe_gather_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(x8), sx, slot_token, offs, n_local,
                                                K, reinterpret_cast<uint8_t*>(x8p), sxp, max_slots);
  return static_cast<int>(cudaGetLastError());
}

int ulc_moe_combine(const void* y, const int32_t* inv_slot, const float* gate, const void* shared, int B, int topk,
                    int H, void* out, void* const* peer_out, int n_peers, int rows_per_peer,
                    const int32_t* shared_slot0, int shared_lo, int shared_n, cudaStream_t stream) {
  if (B <= 0) return 0;
  if ((H % 8) || topk > 8 || n_peers < 0 || n_peers > 8 || rows_per_peer < 0) return -kErrUnsupported;
  if (rows_per_peer > 0 && (B + rows_per_peer - 1) / rows_per_peer > n_peers) return -kErrUnsupported;
  PeerOut po;
  po.n = n_peers;
  for (int r = 0; r < 8; ++r) po.p[r] = r < n_peers ? peer_out[r] : nullptr;
  // threads: the row's 16-byte units split evenly over as few steps as 512 threads allow
  const int units = H / 8, steps = (units + 511) / 512;
  const int threads = (((units + steps - 1) / steps) + 31) / 32 * 32;
  moe_combine_kernel<<<B, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y), inv_slot, gate,
                                            reinterpret_cast<const __nv_bfloat16*>(shared), topk, H,
                                            reinterpret_cast<__nv_bfloat16*>(out), po, rows_per_peer, shared_slot0,
                                            shared_lo, shared_n);
  return static_cast<int>(cudaGetLastError());
}

// Stores n_seg local segments (src[i], nbytes[i], multiples of 16) at byte offsets dst_off[i]
// of every buffer in peer_base.
int ulc_peer_put(const void* const* src, const long long* dst_off, const long long* nbytes, int n_seg,
                 void* const* peer_base, int n_peers, cudaStream_t stream) {
  if (n_seg <= 0 || n_peers <= 0) return 0;
  if (n_seg > 4 || n_peers > 8) return -kErrUnsupported;
  PutSegs segs;
  segs.n = n_seg;
  long long most = 0;
  for (int i = 0; i < n_seg; ++i) {
    if ((nbytes[i] % 16) || (dst_off[i] % 16) || (reinterpret_cast<uintptr_t>(src[i]) % 16)) return -kErrUnsupported;
    segs.src[i] = reinterpret_cast<const uint4*>(src[i]);
    segs.dst_off[i] = dst_off[i];
    segs.units[i] = nbytes[i] / 16;
    most = segs.units[i] > most ? segs.units[i] : most;
  }
  PeerOut po;
  po.n = n_peers;
  for (int r = 0; r < 8; ++r) po.p[r] = r < n_peers ? peer_base[r] : nullptr;
  int blocks = static_cast<int>((most + 255) / 256);
  blocks = blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks);
  peer_put_kernel<<<dim3(blocks, n_peers), 256, 0, stream>>>(segs, po);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
