// Sum of a float buffer over the GPUs of an NVSwitch domain with multimem instructions:
// the view-parallel job's gradient all-reduce (no counterpart in the reference, which is
// single-GPU).
//
// Every rank holds the buffer at the same offset of a symmetric allocation that is also
// bound to an NVLink multicast object; `mc` is the multicast address of that buffer.  The
// range is cut into one slice per rank.  A rank pulls the sum of its slice with
// multimem.ld_reduce (the switch reads the 16 bytes from every GPU and adds them on the way)
// and writes it back with multimem.st (the switch stores it to every GPU): per GPU, (N-1)/N
// of the range leaves through its links and (N-1)/N comes back, once.
//
// The kernel waits for nothing.  The caller orders it: every rank must have finished writing
// the range before any rank launches this (a barrier among the ranks on the launching
// streams), and every rank's launch must have finished before any rank reads the sums.
#include "rm_common.cuh"

namespace rm {

constexpr int kSumThreads = 256;
constexpr int kSumUnroll = 4;

__device__ __forceinline__ float4 multimem_load_sum(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ void multimem_store(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// 16-byte vectors [v_begin, v_end) of the buffer at multicast address mc
__global__ void __launch_bounds__(kSumThreads)
k_multimem_sum(float* __restrict__ mc, int64_t v_begin, int64_t v_end) {
  const int64_t stride = (int64_t)gridDim.x * kSumThreads;
  int64_t i = v_begin + (int64_t)blockIdx.x * kSumThreads + threadIdx.x;
  for (; i + (kSumUnroll - 1) * stride < v_end; i += kSumUnroll * stride) {
    float4 v[kSumUnroll];
#pragma unroll
    for (int u = 0; u < kSumUnroll; ++u) v[u] = multimem_load_sum(mc + 4 * (i + u * stride));
#pragma unroll
    for (int u = 0; u < kSumUnroll; ++u) multimem_store(mc + 4 * (i + u * stride), v[u]);
  }
  for (; i < v_end; i += stride) multimem_store(mc + 4 * i, multimem_load_sum(mc + 4 * i));
}

}  // namespace rm

int rm_launch_multimem_sum(float* mc, int64_t float_begin, int64_t float_end, int rank, int world,
                           cudaStream_t st) {
  const int64_t vb = float_begin / 4, ve = float_end / 4;
  const int64_t per = (ve - vb + world - 1) / world;
  const int64_t b = vb + per * rank, e = b + per < ve ? b + per : ve;
  if (e <= b) return RM_OK;
  int dev = 0, sms = 0;
  RM_CUDA_CHECK(cudaGetDevice(&dev));
  RM_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t want = (e - b + rm::kSumThreads * rm::kSumUnroll - 1) / (rm::kSumThreads * rm::kSumUnroll);
  const unsigned blocks = (unsigned)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
  RmProfScope prof("k_multimem_sum", st);
  rm_count_launch(), rm::k_multimem_sum<<<blocks, rm::kSumThreads, 0, st>>>(mc, b, e);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}
