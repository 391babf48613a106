// Activation transport between source ranks (token owners) and expert owners, plus the
// HBM-bound elementwise stages around the grouped GEMMs.
//
// Dispatch is a PULL: the expert owner reads each routed row from the source rank's staging
// buffer (its own memory at EP1, a CUDA-IPC peer mapping over NVLink otherwise) with 16-byte
// loads and writes it into its own row buffer.  Return is a PUSH done by the GEMM epilogues
// (gemm.cuh, EpiloguePush).  Completion is tracked with monotonically growing generation
// flags, one 128-byte line per (flag kind, peer); nothing is ever reset and every wait is
// bounded.  Reference dataflow: src/cuda/blackwell/fused/impls/routed_bf16.cuh:378-557
// (pull), :1147-1306 (combine); weftmoe/blackwell_backward.py:55-176 (gather, SwiGLU
// backward, return, combine).
#include "kernels.h"
#include "ptx.cuh"
#include "route.h"

namespace wm {

// ------------------------------------------------------------------ flags
__global__ void wait_flags_kernel(const int* flags, int world, Gen generation, int* status,
                                  int* split_on_fail, long long budget) {
  bool ok = true;
  if (threadIdx.x < world)
    ok = wait_flag_ge(flags + threadIdx.x * kFlagStride, generation.value(), status, budget);
  // A wait ran out (now or earlier in this call: the status word is sticky until the host polls it):
  // empty the owner schedule's ranges so that no later kernel of the call follows indices that may
  // never have arrived.
  const bool failed = __any_sync(0xffffffffu, !ok) || *status != 0;
  if (failed && split_on_fail != nullptr)
    for (int i = threadIdx.x; i < kSplitWords; i += blockDim.x) split_on_fail[i] = 0;
}
__global__ void signal_peers_kernel(PeerInts group, int world, int slot, Gen gen) {
  const int generation = gen.value();
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(group.p[threadIdx.x] + slot * kFlagStride, generation);
  }
}
int wait_flags(const int* flags, int world, Gen generation, int* status, int* split_on_fail,
               cudaStream_t stream) {
  wait_flags_kernel<<<1, 32, 0, stream>>>(flags, world, generation, status, split_on_fail,
                                          flag_wait_budget());
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}
int signal_peers(const PeerInts& group, int world, int slot, Gen generation, cudaStream_t stream) {
  signal_peers_kernel<<<1, 32, 0, stream>>>(group, world, slot, generation);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ row copies
// What a warp does with one row: copy `src` to `dst`, write zeros (src == nullptr), or nothing
// (dst == nullptr).
struct RowJob {
  const uint4* src;
  uint4* dst;
};
// One warp serves two rows at a time: every lane first issues all its loads of both rows (up to eight
// 16-byte loads per lane: what covers the latency of a peer's memory over NVLink), then stores them.
__device__ __forceinline__ void run_row_jobs(const RowJob& a, const RowJob& b, int vecs, int lane) {
  constexpr int kDepth = 4;
  for (int c = lane; c < vecs; c += 32 * kDepth) {
    uint4 va[kDepth], vb[kDepth];
#pragma unroll
    for (int j = 0; j < kDepth; ++j) {
      const int i = c + 32 * j;
      va[j] = (a.src != nullptr && i < vecs) ? a.src[i] : make_uint4(0, 0, 0, 0);
      vb[j] = (b.src != nullptr && i < vecs) ? b.src[i] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < kDepth; ++j) {
      const int i = c + 32 * j;
      if (a.dst != nullptr && i < vecs) a.dst[i] = va[j];
      if (b.dst != nullptr && i < vecs) b.dst[i] = vb[j];
    }
  }
}

// The source row of a routed row: origin = src_rank * cap * top_k + token * top_k + sorted_slot.
__device__ __forceinline__ const uint4* source_row(const PeerConstRows& stage, int org, int cap, int top_k,
                                                   int hidden) {
  const int src = org / (cap * top_k);
  const int token = (org - src * cap * top_k) / top_k;
  return reinterpret_cast<const uint4*>(stage.p[src] + static_cast<size_t>(token) * hidden);
}

__global__ void gather_rows_kernel(OwnerRows o, int rank, int e_local, int world, int row_capacity,
                                   int cap, int top_k, int hidden, PeerConstRows stage,
                                   const int* __restrict__ meta_origin,
                                   const float* __restrict__ meta_prob,
                                   const int* __restrict__ meta_primary,
                                   __nv_bfloat16* __restrict__ rows_out,
                                   int* __restrict__ origin_out, float* __restrict__ prob_out,
                                   int* __restrict__ primary_out) {
  const int rows = *o.rows.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = hidden / 8;
  // Looks row r up, writes its origin / prob / primary words and says what to copy.
  auto job_of = [&](int r) -> RowJob {
    if (r >= rows) return RowJob{nullptr, nullptr};
    const int l = o.tile_group[r >> 7];
    const int within = r - o.padded_start[l];
    const bool live = within < o.expert_total[rank * e_local + l];
    uint4* dst = reinterpret_cast<uint4*>(rows_out + static_cast<size_t>(r) * hidden);
    // An origin word outside [0, world * cap * top_k) can only be a word its source never wrote (a
    // source that failed its own plan): the row is treated as padding.
    const int org = live ? meta_origin[r] : -1;
    if (live && org >= 0 && org < world * cap * top_k) {
      int first = meta_primary ? meta_primary[r] : r;
      if (first < 0 || first >= row_capacity) first = r;
      if (lane == 0) {
        origin_out[r] = org;
        prob_out[r] = meta_prob[r];
        if (primary_out) primary_out[r] = first;
      }
      // duplicates of a token inside this rank are copied locally afterwards
      return first == r ? RowJob{source_row(stage, org, cap, top_k, hidden), dst} : RowJob{nullptr, nullptr};
    }
    if (lane == 0) {
      origin_out[r] = -1;
      prob_out[r] = 0.0f;
      if (primary_out) primary_out[r] = r;
    }
    return RowJob{nullptr, dst};
  };
  for (int r = *o.rows.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += 2 * warps)
    run_row_jobs(job_of(r), job_of(r + warps), vecs, lane);
}

__global__ void gather_by_origin_kernel(DeviceRange range, const int* __restrict__ origin,
                                        const int* __restrict__ primary, int world, int cap, int top_k,
                                        int hidden, PeerConstRows stage,
                                        __nv_bfloat16* __restrict__ rows_out) {
  const int rows = *range.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = hidden / 8;
  auto job_of = [&](int r) -> RowJob {
    if (r >= rows) return RowJob{nullptr, nullptr};
    const int org = origin[r];
    uint4* dst = reinterpret_cast<uint4*>(rows_out + static_cast<size_t>(r) * hidden);
    if (org < 0 || org >= world * cap * top_k) return RowJob{nullptr, dst};      // padding: zeros
    if (primary != nullptr && primary[r] != r) return RowJob{nullptr, nullptr};  // copied locally afterwards
    return RowJob{source_row(stage, org, cap, top_k, hidden), dst};
  };
  for (int r = *range.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += 2 * warps)
    run_row_jobs(job_of(r), job_of(r + warps), vecs, lane);
}

__global__ void copy_duplicate_rows_kernel(DeviceRange range, const int* __restrict__ primary,
                                           int hidden, __nv_bfloat16* __restrict__ rows_out) {
  const int rows = *range.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = hidden / 8;
  auto job_of = [&](int r) -> RowJob {
    if (r >= rows) return RowJob{nullptr, nullptr};
    const int first = primary[r];
    if (first == r || first < 0) return RowJob{nullptr, nullptr};
    return RowJob{reinterpret_cast<const uint4*>(rows_out + static_cast<size_t>(first) * hidden),
                  reinterpret_cast<uint4*>(rows_out + static_cast<size_t>(r) * hidden)};
  };
  for (int r = *range.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += 2 * warps)
    run_row_jobs(job_of(r), job_of(r + warps), vecs, lane);
}

int gather_rows(const OwnerRows& o, int rank, int e_local, int world, int row_capacity, int cap, int top_k,
                int hidden,
                const PeerConstRows& stage, const int* meta_origin, const float* meta_prob,
                const int* meta_primary, __nv_bfloat16* rows_out, int* origin_out, float* prob_out,
                int* primary_out, int ctas, cudaStream_t stream) {
  gather_rows_kernel<<<ctas, 256, 0, stream>>>(o, rank, e_local, world, row_capacity, cap, top_k, hidden, stage,
                                                  meta_origin, meta_prob, meta_primary, rows_out,
                                                  origin_out, prob_out, primary_out);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}
int gather_by_origin(DeviceRange rows, const int* origin, const int* primary, int world, int cap, int top_k,
                     int hidden, const PeerConstRows& stage, __nv_bfloat16* rows_out, int ctas,
                     cudaStream_t stream) {
  gather_by_origin_kernel<<<ctas, 256, 0, stream>>>(rows, origin, primary, world, cap, top_k, hidden, stage,
                                                   rows_out);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}
int copy_duplicate_rows(DeviceRange rows, const int* primary, int hidden, __nv_bfloat16* rows_out,
                        int ctas, cudaStream_t stream) {
  copy_duplicate_rows_kernel<<<ctas, 256, 0, stream>>>(rows, primary, hidden, rows_out);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ combine
// One CTA per token; each thread owns 8 consecutive columns.  Contributions are added in
// ascending combine position with sequential FP32 adds: the order defines the bits
// (reference: routed_bf16.cuh:1209-1306, fused/ptx/utils.cuh:70-79).
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ mailbox,
                                    const int* __restrict__ sorted_expert, int cap, int top_k,
                                    int hidden, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  const int vecs = hidden / 8;
  for (int c = threadIdx.x; c < vecs; c += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    // Four contributions are loaded at a time (their latencies overlap) and then added one after the
    // other; a slot without a contribution adds +0.0, which leaves every bit of the sum as it was.
    for (int j0 = 0; j0 < top_k; j0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = j0 + i;
        const bool live = j < top_k && sorted_expert[t * top_k + j] >= 0;
        v[i] = live ? *reinterpret_cast<const uint4*>(mailbox + (static_cast<size_t>(j) * cap + t) * hidden + c * 8)
                    : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[2 * k] += __uint_as_float(w[k] << 16);
          acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
        }
      }
    }
    uint4 r;
    r.x = pack_bf16x2(acc[0], acc[1]);
    r.y = pack_bf16x2(acc[2], acc[3]);
    r.z = pack_bf16x2(acc[4], acc[5]);
    r.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + c * 8) = r;
  }
}
int combine_rows(const __nv_bfloat16* mailbox, const int* sorted_expert, int tokens, int cap,
                 int top_k, int hidden, __nv_bfloat16* out, cudaStream_t stream) {
  if (tokens == 0) return 0;
  const int threads = hidden / 8 >= 256 ? 256 : ((hidden / 8 + 31) / 32 * 32);
  combine_rows_kernel<<<tokens, threads, 0, stream>>>(mailbox, sorted_expert, cap, top_k, hidden,
                                                      out);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

__global__ void unpermute_dgates_kernel(const float* __restrict__ box,
                                        const int* __restrict__ sorted_slot,
                                        const int* __restrict__ sorted_expert, int n, int top_k,
                                        float* __restrict__ dgates) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int t = i / top_k;
  dgates[t * top_k + sorted_slot[i]] = sorted_expert[i] >= 0 ? box[i] : 0.0f;
}
int unpermute_dgates(const float* dgate_box, const int* sorted_slot, const int* sorted_expert,
                     int tokens, int top_k, float* dgates, cudaStream_t stream) {
  const int n = tokens * top_k;
  if (n == 0) return 0;
  unpermute_dgates_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dgate_box, sorted_slot,
                                                               sorted_expert, n, top_k, dgates);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ SwiGLU backward
// One warp per routed row (reference math: weftmoe/blackwell_backward.py:81-113):
//   sig = sigmoid(a); silu = a*sig; U = bf16(silu*b*p)
//   dA = bf16(dU*p*b*sig*(1+a*(1-sig))); dB = bf16(dU*p*silu); dprob = sum_i dU_i*silu_i*b_i
// The row sum uses a fixed lane->column assignment and a fixed shuffle tree: deterministic.
__global__ void swiglu_backward_kernel(DeviceRange range, const __nv_bfloat16* __restrict__ ab,
                                       const __nv_bfloat16* __restrict__ du,
                                       const float* __restrict__ prob,
                                       const int* __restrict__ origin, int inter, int cap,
                                       int top_k, __nv_bfloat16* __restrict__ u,
                                       __nv_bfloat16* __restrict__ dab, PeerFloats dgate_box) {
  const int rows = *range.end;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vecs = inter / 8;
  for (int r = *range.begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    const float p = prob[r];
    const uint4* pa = reinterpret_cast<const uint4*>(ab + static_cast<size_t>(r) * 2 * inter);
    const uint4* pb = pa + vecs;
    const uint4* pdu = reinterpret_cast<const uint4*>(du + static_cast<size_t>(r) * inter);
    uint4* pu = reinterpret_cast<uint4*>(u + static_cast<size_t>(r) * inter);
    uint4* pda = reinterpret_cast<uint4*>(dab + static_cast<size_t>(r) * 2 * inter);
    uint4* pdb = pda + vecs;
    float dsum = 0.0f;
    for (int c = lane; c < vecs; c += 32) {
      const uint4 va = pa[c], vb = pb[c], vd = pdu[c];
      const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w},
                     wd[4] = {vd.x, vd.y, vd.z, vd.w};
      uint32_t ou[4], oa[4], ob[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float res_u[2], res_a[2], res_b[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float a = __uint_as_float(h ? (wa[k] & 0xffff0000u) : (wa[k] << 16));
          const float b = __uint_as_float(h ? (wb[k] & 0xffff0000u) : (wb[k] << 16));
          const float d = __uint_as_float(h ? (wd[k] & 0xffff0000u) : (wd[k] << 16));
          const float sig = 1.0f / (1.0f + __expf(-a));
          const float silu = a * sig;
          const float act = silu * b;
          res_u[h] = act * p;
          res_a[h] = d * p * b * (sig * (1.0f + a * (1.0f - sig)));
          res_b[h] = d * p * silu;
          dsum += d * act;
        }
        ou[k] = pack_bf16x2(res_u[0], res_u[1]);
        oa[k] = pack_bf16x2(res_a[0], res_a[1]);
        ob[k] = pack_bf16x2(res_b[0], res_b[1]);
      }
      pu[c] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      pda[c] = make_uint4(oa[0], oa[1], oa[2], oa[3]);
      pdb[c] = make_uint4(ob[0], ob[1], ob[2], ob[3]);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, d);
    const int org = origin[r];
    if (lane == 0 && org >= 0) {
      const int per = cap * top_k;
      const int src = org / per;
      dgate_box.p[src][org - src * per] = dsum;
    }
  }
}
// dprob of a row = its partial sums over the column blocks of the fused dU epilogue, added in block
// order; sent to the source rank's dprob box like swiglu_backward does.
__global__ void dprob_finish_kernel(DeviceRange range, const float* __restrict__ part, int blocks,
                                    int row_capacity, const int* __restrict__ origin, int cap, int top_k,
                                    PeerFloats dgate_box) {
  const int rows = *range.end;
  for (int r = *range.begin + blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const int org = origin[r];
    if (org < 0) continue;
    float sum = 0.0f;
    for (int t = 0; t < blocks; ++t) sum += part[static_cast<size_t>(t) * row_capacity + r];
    const int per = cap * top_k;
    const int src = org / per;
    dgate_box.p[src][org - src * per] = sum;
  }
}
int dprob_finish(DeviceRange rows, const float* part, int blocks, int row_capacity, const int* origin, int cap,
                 int top_k, const PeerFloats& dgate_box, cudaStream_t stream) {
  dprob_finish_kernel<<<256, 256, 0, stream>>>(rows, part, blocks, row_capacity, origin, cap, top_k, dgate_box);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

int swiglu_backward(DeviceRange rows, const __nv_bfloat16* ab, const __nv_bfloat16* du,
                    const float* prob, const int* origin, int inter, int cap, int top_k,
                    __nv_bfloat16* u, __nv_bfloat16* dab, const PeerFloats& dgate_box, int sms,
                    cudaStream_t stream) {
  swiglu_backward_kernel<<<sms * 8, 256, 0, stream>>>(rows, ab, du, prob, origin, inter, cap,
                                                      top_k, u, dab, dgate_box);
  count_launch();
  WM_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace wm
