// Per-tet feature activation fused into one pass: the step that produces the
// [T,7] cell values the rasterizer consumes when a frozen model is rendered
// (utils/model_util.py:81-105 activate_output with offset_normalize :81-91 and
// compute_vertex_colors_from_field :63-79; utils/eval_sh_py.py:121-179 eval_sh;
// call sites tile_benchmark.py:62-67, models/frozen.py:216-223).
//
// The reference evaluates this with about twenty torch kernels and as many
// [T,*] temporaries; here one thread per tet reads its inputs once (about
// 100 + 12*K bytes, K SH coefficients per channel beyond degree 0) and writes
// the 28-byte feature row.  Forward only: it serves the no-grad rendering path.

#include <cuda_fp16.h>

#include "rm_common.cuh"

namespace rm {

__device__ __forceinline__ float safe_div_torch(float n, float d) {
  // utils/safe_math.py:146-158: 0 where |d| < tiny, else clamp(n / d, min, max)
  const float tiny = 1.17549435e-38f, big = 3.40282347e+38f;
  if (fabsf(d) < tiny) return 0.0f;
  return fminf(fmaxf(n / d, -big), big);
}

__device__ __forceinline__ void act_cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ float sh_load(const float* p) { return *p; }
__device__ __forceinline__ float sh_load(const __half* p) { return __half2float(*p); }

constexpr int kActThreads = 128;

// Shared memory: the block's slab of SH coefficients (kActThreads * n_rest * 3 values, contiguous in
// global memory, copied with 16-byte loads) followed by the block's output rows (kActThreads * 7 floats,
// written back with 16-byte stores).  A thread then reads its own row from shared memory.
template <typename SH>
__global__ void __launch_bounds__(kActThreads)
k_activate_output(const float* __restrict__ camera_center, const float* __restrict__ density,
                  const float* __restrict__ rgb, const float* __restrict__ grd, const SH* __restrict__ sh,
                  const int32_t* __restrict__ indices, const float* __restrict__ circumcenters,
                  const float* __restrict__ vertices, int64_t T, int deg, int n_rest, float* __restrict__ features) {
  extern __shared__ uint4 smem_act[];
  const int64_t first = (int64_t)blockIdx.x * kActThreads;
  const int rows = (int)min((int64_t)kActThreads, T - first);
  const int row_vals = n_rest * 3;
  SH* sh_s = reinterpret_cast<SH*>(smem_act);
  const int slab_bytes = kActThreads * row_vals * (int)sizeof(SH);  // a multiple of 16
  float* out_s = reinterpret_cast<float*>(reinterpret_cast<char*>(smem_act) + slab_bytes);
  if (deg > 0) {  // start the slab copy; it lands while the geometry below is fetched and evaluated
    const SH* src = sh + first * row_vals;
    if (rows == kActThreads && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      const uint4* src4 = reinterpret_cast<const uint4*>(src);
      for (int i = threadIdx.x; i < slab_bytes / 16; i += kActThreads) act_cp_async16(smem_act + i, src4 + i);
    } else {
      for (int i = threadIdx.x; i < rows * row_vals; i += kActThreads) sh_s[i] = src[i];
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  const int64_t g = first + threadIdx.x;
  const bool live = g < T;
  const float C0 = 0.28209479177387814f;
  f3 res = {0.f, 0.f, 0.f}, ng = {0.f, 0.f, 0.f};
  float x = 0.f, y = 0.f, z = 0.f, dens = 0.f;
  if (live) {
    const int4 id = __ldg(reinterpret_cast<const int4*>(indices) + g);
    const f3 v0 = load3(vertices, id.x), v1 = load3(vertices, id.y), v2 = load3(vertices, id.z),
             v3 = load3(vertices, id.w);
    const f3 cc = load3(circumcenters, g);
    const f3 c = load3(rgb, g);
    f3 gr = load3(grd, g);
    // offset_normalize: gradient scaled by the smallest colour channel and by 1 / circumradius
    const float cmin = fminf(c.x, fminf(c.y, c.z));
    gr = gr * cmin;
    const f3 r0 = v0 - cc;
    const float radius = sqrtf(r0.x * r0.x + r0.y * r0.y + r0.z * r0.z);
    ng = f3{safe_div_torch(gr.x, radius), safe_div_torch(gr.y, radius), safe_div_torch(gr.z, radius)};
    dens = __ldg(density + g);
    // colour at vertex 0: base + normed_grd . (v0 - circumcenter), the same offset on all channels
    const float off = ng.x * r0.x + ng.y * r0.y + ng.z * r0.z;
    const f3 base_v0 = {c.x + off, c.y + off, c.z + off};
    // eval_sh at the direction from the camera to the tet centroid
    const f3 sh0 = {(base_v0.x - 0.5f) / C0, (base_v0.y - 0.5f) / C0, (base_v0.z - 0.5f) / C0};  // RGB2SH
    res = f3{C0 * sh0.x + 0.5f, C0 * sh0.y + 0.5f, C0 * sh0.z + 0.5f};
    if (deg > 0) {
      const f3 cam = {__ldg(camera_center), __ldg(camera_center + 1), __ldg(camera_center + 2)};
      const f3 mean = {(v0.x + v1.x + v2.x + v3.x) / 4.0f, (v0.y + v1.y + v2.y + v3.y) / 4.0f,
                       (v0.z + v1.z + v2.z + v3.z) / 4.0f};
      f3 dir = mean - cam;
      const float nrm = fmaxf(sqrtf(dir.x * dir.x + dir.y * dir.y + dir.z * dir.z), 1e-8f);  // F.normalize eps
      x = dir.x / nrm, y = dir.y / nrm, z = dir.z / nrm;
    }
  }
  if (deg > 0) {
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();
  }
  if (live) {
    if (deg > 0) {
      const SH* s = sh_s + threadIdx.x * row_vals;
      auto coef = [&](int k) -> f3 { return {sh_load(s + 3 * k), sh_load(s + 3 * k + 1), sh_load(s + 3 * k + 2)}; };
      auto axpy = [&](float a, f3 b) { res = {res.x + a * b.x, res.y + a * b.y, res.z + a * b.z}; };
      axpy(-0.4886025119029199f * y, coef(0));
      axpy(0.4886025119029199f * z, coef(1));
      axpy(-0.4886025119029199f * x, coef(2));
      if (deg > 1) {
        const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
        axpy(1.0925484305920792f * xy, coef(3));
        axpy(-1.0925484305920792f * yz, coef(4));
        axpy(0.31539156525252005f * (2.0f * zz - xx - yy), coef(5));
        axpy(-1.0925484305920792f * xz, coef(6));
        axpy(0.5462742152960396f * (xx - yy), coef(7));
        if (deg > 2) {
          axpy(-0.5900435899266435f * y * (3.0f * xx - yy), coef(8));
          axpy(2.890611442640554f * xy * z, coef(9));
          axpy(-0.4570457994644658f * y * (4.0f * zz - xx - yy), coef(10));
          axpy(0.3731763325901154f * z * (2.0f * zz - 3.0f * xx - 3.0f * yy), coef(11));
          axpy(-0.4570457994644658f * x * (4.0f * zz - xx - yy), coef(12));
          axpy(1.445305721320277f * z * (xx - yy), coef(13));
          axpy(-0.5900435899266435f * x * (xx - 3.0f * yy), coef(14));
          if (deg > 3) {
            axpy(2.5033429417967046f * xy * (xx - yy), coef(15));
            axpy(-1.7701307697799304f * yz * (3.0f * xx - yy), coef(16));
            axpy(0.9461746957575601f * xy * (7.0f * zz - 1.0f), coef(17));
            axpy(-0.6690465435572892f * yz * (7.0f * zz - 3.0f), coef(18));
            axpy(0.10578554691520431f * (zz * (35.0f * zz - 30.0f) + 3.0f), coef(19));
            axpy(-0.6690465435572892f * xz * (7.0f * zz - 3.0f), coef(20));
            axpy(0.47308734787878004f * (xx - yy) * (7.0f * zz - 1.0f), coef(21));
            axpy(-1.7701307697799304f * xz * (xx - 3.0f * yy), coef(22));
            axpy(0.6258357354491761f * (xx * (xx - 3.0f * yy) - yy * (3.0f * xx - yy)), coef(23));
          }
        }
      }
    }
    // softplus with beta = 10 (torch: linear above beta*x = 20)
    auto softplus10 = [](float v) { return 10.0f * v > 20.0f ? v : log1pf(expf(10.0f * v)) / 10.0f; };
    float* o = out_s + 7 * threadIdx.x;
    o[0] = dens;
    o[1] = softplus10(res.x);
    o[2] = softplus10(res.y);
    o[3] = softplus10(res.z);
    o[4] = ng.x;
    o[5] = ng.y;
    o[6] = ng.z;
  }
  __syncthreads();
  float* dst = features + 7 * first;  // 7 * 128 floats per block: 16-byte aligned whenever `features` is
  if (rows == kActThreads && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    for (int i = threadIdx.x; i < kActThreads * 7 / 4; i += kActThreads)
      reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(out_s)[i];
  } else {
    for (int i = threadIdx.x; i < rows * 7; i += kActThreads) dst[i] = out_s[i];
  }
}

}  // namespace rm

int rm_launch_activate(const float* camera_center, const float* density, const float* rgb, const float* grd,
                       const void* sh, int sh_is_half, const int32_t* indices, const float* circumcenters,
                       const float* vertices, int64_t T, int deg, int n_rest, float* features, cudaStream_t st) {
  if (T == 0) return RM_OK;
  const unsigned blocks = (unsigned)((T + rm::kActThreads - 1) / rm::kActThreads);
  const size_t smem = (size_t)rm::kActThreads * n_rest * 3 * (sh_is_half ? 2 : 4) + rm::kActThreads * 7 * sizeof(float);
  RmProfScope prof("k_activate_output", st);
  if (sh_is_half)
    rm_count_launch(), rm::k_activate_output<__half><<<blocks, rm::kActThreads, smem, st>>>(
        camera_center, density, rgb, grd, static_cast<const __half*>(sh), indices, circumcenters, vertices, T, deg,
        n_rest, features);
  else
    rm_count_launch(), rm::k_activate_output<float><<<blocks, rm::kActThreads, smem, st>>>(
        camera_center, density, rgb, grd, static_cast<const float*>(sh), indices, circumcenters, vertices, T, deg,
        n_rest, features);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}
