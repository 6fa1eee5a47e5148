// extern "C" entry points of librm_b200.so: argument checks, device binding and
// the launch sequence of each stage.  See include/rm_b200.h for the contract.

#include <stdio.h>
#include <string.h>

#include "rm_common.cuh"

// launchers defined in the kernel translation units
int rm_launch_project(const int32_t*, int64_t, const float*, int64_t, const RmCamera*, int32_t*, int32_t*, float*,
                      float*, uint32_t*, uint32_t*, int32_t*, RmBinInfo*, cudaStream_t);
int rm_launch_vertex_backward(const int32_t*, const float*, int64_t, const RmCamera*, const int32_t*, const float*,
                              const float*, float*, cudaStream_t);
size_t rm_bin_layout_bytes(int64_t, int64_t);
int rm_launch_bin_prepare(int64_t, const RmCamera*, void*, size_t, uint32_t**, uint32_t**, int32_t**, RmBinInfo*,
                          cudaStream_t);
int rm_launch_bin_finish(int64_t, const RmCamera*, const int32_t*, int32_t*, RmBinInfo*, void*, cudaStream_t);
int rm_launch_build_lists(const int32_t*, const int32_t*, int64_t, const RmCamera*, int64_t, int64_t, void*, void*, size_t,
                          int32_t*, cudaStream_t);
size_t rm_list_plan_bytes(int64_t, int, int);
int rm_launch_pack(const int32_t*, const float*, const float*, int64_t, int64_t, const RmCamera*, const int32_t*,
                   float*, cudaStream_t);
int rm_launch_forward(const int32_t*, const int32_t*, const float*, const RmCamera*, const float*, float*, float*,
                      int32_t*, const RmHitList*, cudaStream_t);
int rm_launch_forward_constant_color(const int32_t*, const int32_t*, const float*, const RmCamera*, float, float,
                                     float*, float*, int32_t*, cudaStream_t);
int rm_launch_backward_integrate(const int32_t*, const float*, const RmCamera*, const float*, const float*, const float*,
                                 const RmHitList*, const float*, const float*, int64_t, int64_t, float*, float*,
                                 cudaStream_t);
int rm_launch_backward_finish(const int32_t*, const float*, const float*, int64_t, int64_t, const RmCamera*,
                              const float*, const RmHitList*, float*, float*, cudaStream_t);

int rm_launch_tet_err(const int32_t*, const int32_t*, const float*, const RmCamera*, const float*, const float*,
                      int64_t, float*, int32_t*, cudaStream_t);
int rm_launch_backward_constant_color(const int32_t*, const int32_t*, const float*, const RmCamera*, float, float,
                                      const float*, const float*, const int32_t*, const float*, const float*, int64_t,
                                      int64_t, float*, uint8_t*, float*, cudaStream_t);

int rm_launch_multimem_sum(float*, int64_t, int64_t, int, int, cudaStream_t);
int rm_launch_activate(const float*, const float*, const float*, const float*, const void*, int, const int32_t*,
                       const float*, const float*, int64_t, int, int, float*, cudaStream_t);

void rm_debug_extent_raster(int which, long long n);

static thread_local char g_last_error[256] = "";

// ---- optional per-kernel timing ---------------------------------------------
#include <mutex>
#include <vector>
namespace {
struct ProfRec {
  const char* name;
  cudaEvent_t a, b;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRec> g_prof;
thread_local int g_prof_open = -1;
}  // namespace

void rm_prof_begin(const char* name, cudaStream_t st) {
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  ProfRec r{name, nullptr, nullptr};
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
  cudaEventRecord(r.a, st);
  g_prof.push_back(r);
  g_prof_open = (int)g_prof.size() - 1;
}
void rm_prof_end(cudaStream_t st) {
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof_open >= 0 && g_prof_open < (int)g_prof.size()) cudaEventRecord(g_prof[g_prof_open].b, st);
  g_prof_open = -1;
}

#include <atomic>
static std::atomic<long long> g_launches{0};
void rm_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void rm_set_last_cuda_error(cudaError_t e, const char* file, int line) {
  snprintf(g_last_error, sizeof(g_last_error), "CUDA error %d (%s) at %s:%d", (int)e, cudaGetErrorString(e), file,
           line);
}

// Make the device that owns `device_ptr` current on this thread (the forward
// pass runs on the caller's main thread, the backward pass on an autograd
// worker thread).
int rm_bind_device(const void* device_ptr) {
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, device_ptr);
  if (e != cudaSuccess) {
    rm_set_last_cuda_error(e, __FILE__, __LINE__);
    return RM_ERR_CUDA;
  }
  if (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged) {
    snprintf(g_last_error, sizeof(g_last_error), "pointer %p is not device memory", device_ptr);
    return RM_ERR_INVALID_ARG;
  }
  int cur = -1;
  RM_CUDA_CHECK(cudaGetDevice(&cur));
  if (cur != a.device) RM_CUDA_CHECK(cudaSetDevice(a.device));
  return RM_OK;
}

int rm_check_cam(const RmCamera* c) {
  if (!c || !c->world_view_transform || !c->K || !c->cam_pos || !c->distortion_params) return RM_ERR_INVALID_ARG;
  if (c->image_height <= 0 || c->image_width <= 0 || c->tile_height <= 0 || c->tile_width <= 0)
    return RM_ERR_INVALID_ARG;
  if (c->grid_height != (c->image_height + c->tile_height - 1) / c->tile_height ||
      c->grid_width != (c->image_width + c->tile_width - 1) / c->tile_width)
    return RM_ERR_INVALID_ARG;
  if (c->tile_row_begin < 0 || c->tile_row_end > c->grid_height || c->tile_row_begin > c->tile_row_end)
    return RM_ERR_INVALID_ARG;
  if ((int64_t)c->grid_height * c->grid_width > 0x7fffffffll) return RM_ERR_INVALID_ARG;
  return RM_OK;
}
void rm_clear_last_error() { g_last_error[0] = 0; }

extern "C" {

const char* rm_strerror(int code) {
  switch (code) {
    case RM_OK: return "ok";
    case RM_ERR_INVALID_ARG: return g_last_error[0] ? g_last_error : "invalid argument";
    case RM_ERR_CUDA: return g_last_error[0] ? g_last_error : "CUDA error";
    case RM_ERR_TOO_MANY_KEYS: return "more than 2^31-1 (tile, tet) pairs";
    case RM_ERR_WORKSPACE: return "workspace too small or misaligned";
    case RM_ERR_STATIC_SCRATCH:
      return "n_tets exceeds RM_STATIC_SCRATCH_MAX_TETS (131072): use rm_backward with a caller-provided scratch";
    default: return "unknown error";
  }
}

int rm_version(void) { return 101; }

int64_t rm_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int rm_debug_bounds_checked(void) {
#ifdef RM_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}
void rm_debug_set_extent(int which, int64_t n) { rm_debug_extent_raster(which, (long long)n); }
uint32_t rm_debug_bounds_status(void) { return rm_bounds_status_raster() | rm_bounds_status_binning(); }

void rm_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_on = on != 0;
}

int rm_profile_read(char* names, size_t names_bytes, float* ms, int max_records) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  int n = 0;
  size_t off = 0;
  if (names && names_bytes) names[0] = 0;
  for (auto& r : g_prof) {
    float t = 0.f;
    if (r.a && r.b && cudaEventSynchronize(r.b) == cudaSuccess) cudaEventElapsedTime(&t, r.a, r.b);
    if (n < max_records) {
      size_t len = strlen(r.name);
      if (names && off + len + 2 <= names_bytes) {
        memcpy(names + off, r.name, len);
        names[off + len] = '\n';
        names[off + len + 1] = 0;
        off += len + 1;
        if (ms) ms[n] = t;
        ++n;
      }
    }
    if (r.a) cudaEventDestroy(r.a);
    if (r.b) cudaEventDestroy(r.b);
  }
  g_prof.clear();
  return n;
}

size_t rm_bin_workspace_bytes(int64_t n_tets, int64_t n_tiles) {
  if (n_tets < 0 || n_tiles < 0) return 0;
  return rm_bin_layout_bytes(n_tets, n_tiles);
}

int rm_project_and_bin(const int32_t* indices, int64_t n_tets, const float* vertices, int64_t n_vertices,
                       const RmCamera* cam, int32_t* tiles_touched, int32_t* rect_tile_space, float* vs_tetra,
                       float* circumcenter, int32_t* tile_ranges, RmBinInfo* info, void* workspace,
                       size_t workspace_bytes, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0 || n_tets > 0x7fffffffll || !info || !tile_ranges || !workspace)
    return RM_ERR_INVALID_ARG;
  if (n_tets > 0 && (!indices || !vertices || !tiles_touched || !rect_tile_space || !vs_tetra || !circumcenter))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(indices) || !rm_aligned16(rect_tile_space) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(workspace);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t *depth_keys, *order_in;
  int32_t* tile_diff;
  rc = rm_launch_bin_prepare(n_tets, cam, workspace, workspace_bytes, &depth_keys, &order_in, &tile_diff, info, st);
  if (rc) return rc;
  rc = rm_launch_project(indices, n_tets, vertices, n_vertices, cam, tiles_touched, rect_tile_space, vs_tetra,
                         circumcenter, depth_keys, order_in, tile_diff, info, st);
  if (rc) return rc;
  return rm_launch_bin_finish(n_tets, cam, rect_tile_space, tile_ranges, info, workspace, st);
}

size_t rm_list_scratch_bytes(int64_t n_region_keys, int grid_height, int grid_width) {
  if (n_region_keys < 0 || grid_height < 1 || grid_width < 1) return 0;
  return rm_list_plan_bytes(n_region_keys, grid_height, grid_width);
}

int rm_build_tile_lists(const int32_t* rect_tile_space, const int32_t* tile_ranges, int64_t n_tets,
                        const RmCamera* cam, int64_t n_keys, int64_t n_region_keys, void* workspace, void* scratch,
                        size_t scratch_bytes, int32_t* sorted_tetra_idx, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_keys < 0 || n_region_keys < 0 || n_tets < 0 || !workspace || !tile_ranges) return RM_ERR_INVALID_ARG;
  if (n_keys > 0x7fffffffll) return RM_ERR_TOO_MANY_KEYS;
  if (n_keys == 0) return RM_OK;
  if (!rect_tile_space || !scratch || !sorted_tetra_idx) return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(rect_tile_space)) return RM_ERR_WORKSPACE;
  rc = rm_bind_device(workspace);
  if (rc) return rc;
  return rm_launch_build_lists(rect_tile_space, tile_ranges, n_tets, cam, n_keys, n_region_keys, workspace, scratch,
                               scratch_bytes, sorted_tetra_idx, static_cast<cudaStream_t>(stream));
}

int rm_pack_records(const int32_t* indices, const float* vertices, const float* cell_values, int64_t n_tets,
                    int64_t n_vertices, const RmCamera* cam, const int32_t* tiles_touched, float* records,
                    void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0) return RM_ERR_INVALID_ARG;
  if (n_tets == 0) return RM_OK;
  if (!indices || !vertices || !cell_values || !records) return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(indices) || !rm_aligned16(records)) return RM_ERR_WORKSPACE;
  rc = rm_bind_device(records);
  if (rc) return rc;
  return rm_launch_pack(indices, vertices, cell_values, n_tets, n_vertices, cam, tiles_touched, records,
                        static_cast<cudaStream_t>(stream));
}

int rm_forward(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
               const RmCamera* cam, const float* ray_jitter, float* output_img, float* distortion_img,
               int32_t* n_contributors, const RmHitList* hits, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (!tile_ranges || !ray_jitter || !output_img || !distortion_img || !n_contributors) return RM_ERR_INVALID_ARG;
  if (hits && (!hits->counts || !hits->ids || !hits->masks || !hits->tet_flags)) return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(output_img) || !rm_aligned16(records) || (reinterpret_cast<uintptr_t>(ray_jitter) & 7) ||
      (reinterpret_cast<uintptr_t>(tile_ranges) & 7))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(output_img);
  if (rc) return rc;
  return rm_launch_forward(sorted_tetra_idx, tile_ranges, records, cam, ray_jitter, output_img, distortion_img,
                           n_contributors, hits, static_cast<cudaStream_t>(stream));
}

int rm_forward_constant_color(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                              const RmCamera* cam, float pre_multi, float ladder_p, float* output_img,
                              float* distortion_img, int32_t* n_contributors, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (!tile_ranges || !output_img || !distortion_img || !n_contributors || ladder_p == 0.0f)
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(output_img) || !rm_aligned16(distortion_img) || !rm_aligned16(records) ||
      (reinterpret_cast<uintptr_t>(tile_ranges) & 7))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(output_img);
  if (rc) return rc;
  return rm_launch_forward_constant_color(sorted_tetra_idx, tile_ranges, records, cam, pre_multi, ladder_p,
                                          output_img, distortion_img, n_contributors,
                                          static_cast<cudaStream_t>(stream));
}

static int check_backward_args(const int32_t* tile_ranges, const float* records, const RmCamera* cam,
                               const float* ray_jitter, const float* output_img, const float* distortion_img,
                               const RmHitList* hits, const float* grad_output_img, const float* grad_distortion_img,
                               int64_t n_tets, int64_t n_vertices, const float* grad_records,
                               const float* vertices_grad) {
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0) return RM_ERR_INVALID_ARG;
  if (!tile_ranges || !ray_jitter || !output_img || !distortion_img || !hits || !hits->counts || !hits->ids ||
      !hits->masks || !hits->tet_flags || !grad_output_img || !grad_distortion_img || !vertices_grad)
    return RM_ERR_INVALID_ARG;
  if (n_tets > 0 && (!grad_records || !records)) return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(output_img) || !rm_aligned16(grad_output_img) || !rm_aligned16(records) ||
      !rm_aligned16(grad_records))
    return RM_ERR_WORKSPACE;
  return RM_OK;
}

int rm_backward_constant_color(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                               const RmCamera* cam, float pre_multi, float ladder_p, const float* output_img,
                               const float* distortion_img, const int32_t* n_contributors,
                               const float* grad_output_img, const float* grad_distortion_img, const int32_t* indices,
                               const float* vertices, const float* cell_values, int64_t n_tets, int64_t n_vertices,
                               float* grad_records, uint8_t* tet_flags, float* vertices_grad, float* cell_values_grad,
                               void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0 || ladder_p == 0.0f) return RM_ERR_INVALID_ARG;
  if (!tile_ranges || !output_img || !distortion_img || !n_contributors || !grad_output_img || !grad_distortion_img ||
      !vertices_grad)
    return RM_ERR_INVALID_ARG;
  if (n_tets > 0 && (!sorted_tetra_idx || !records || !indices || !vertices || !cell_values || !grad_records ||
                     !tet_flags || !cell_values_grad))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(output_img) || !rm_aligned16(distortion_img) || !rm_aligned16(grad_output_img) ||
      !rm_aligned16(grad_distortion_img) || !rm_aligned16(records) || !rm_aligned16(grad_records) ||
      !rm_aligned16(indices))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(vertices_grad);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = rm_launch_backward_constant_color(sorted_tetra_idx, tile_ranges, records, cam, pre_multi, ladder_p, output_img,
                                         distortion_img, n_contributors, grad_output_img, grad_distortion_img, n_tets,
                                         n_vertices, grad_records, tet_flags, vertices_grad, st);
  if (rc) return rc;
  RmHitList flags_only = {nullptr, nullptr, nullptr, tet_flags};
  return rm_launch_backward_finish(indices, vertices, cell_values, 0, n_tets, cam, grad_records, &flags_only,
                                   vertices_grad, cell_values_grad, st);
}

int rm_backward_integrate(const int32_t* tile_ranges, const float* records, const RmCamera* cam,
                          const float* ray_jitter, const float* output_img, const float* distortion_img,
                          const RmHitList* hits, const float* grad_output_img, const float* grad_distortion_img,
                          int64_t n_tets, int64_t n_vertices, float* grad_records, float* vertices_grad, void* stream) {
  g_last_error[0] = 0;
  int rc = check_backward_args(tile_ranges, records, cam, ray_jitter, output_img, distortion_img, hits,
                               grad_output_img, grad_distortion_img, n_tets, n_vertices, grad_records, vertices_grad);
  if (rc) return rc;
  rc = rm_bind_device(vertices_grad);
  if (rc) return rc;
  return rm_launch_backward_integrate(tile_ranges, records, cam, ray_jitter, output_img, distortion_img, hits,
                                      grad_output_img, grad_distortion_img, n_tets, n_vertices, grad_records,
                                      vertices_grad, static_cast<cudaStream_t>(stream));
}

int rm_backward_finish(const int32_t* indices, const float* vertices, const float* cell_values, int64_t tet_begin,
                       int64_t tet_end, int64_t n_tets, const RmCamera* cam, const float* grad_records,
                       const RmHitList* hits, float* vertices_grad, float* cell_values_grad, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (tet_begin < 0 || tet_end < tet_begin || tet_end > n_tets) return RM_ERR_INVALID_ARG;
  if (tet_end == tet_begin) return RM_OK;
  if (!indices || !vertices || !cell_values || !grad_records || !hits || !hits->tet_flags || !vertices_grad ||
      !cell_values_grad)
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(indices) || !rm_aligned16(grad_records)) return RM_ERR_WORKSPACE;
  rc = rm_bind_device(vertices_grad);
  if (rc) return rc;
  return rm_launch_backward_finish(indices, vertices, cell_values, tet_begin, tet_end, cam, grad_records, hits,
                                   vertices_grad, cell_values_grad, static_cast<cudaStream_t>(stream));
}

int rm_backward(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                const RmCamera* cam, const float* ray_jitter, const float* output_img,
                const float* distortion_img, const int32_t* n_contributors, const RmHitList* hits,
                const float* grad_output_img, const float* grad_distortion_img, const int32_t* indices,
                const float* vertices, const float* cell_values, int64_t n_tets, int64_t n_vertices,
                float* grad_records, float* vertices_grad, float* cell_values_grad, void* stream) {
  (void)sorted_tetra_idx;
  (void)n_contributors;  // the hit lists already stop at every pixel's last contributor
  int rc = rm_backward_integrate(tile_ranges, records, cam, ray_jitter, output_img, distortion_img, hits,
                                 grad_output_img, grad_distortion_img, n_tets, n_vertices, grad_records, vertices_grad,
                                 stream);
  if (rc) return rc;
  if (n_tets > 0 && (!indices || !vertices || !cell_values || !cell_values_grad)) return RM_ERR_INVALID_ARG;
  return rm_backward_finish(indices, vertices, cell_values, 0, n_tets, n_tets, cam, grad_records, hits, vertices_grad,
                            cell_values_grad, stream);
}

int rm_multimem_sum(float* multicast_buffer, int64_t float_begin, int64_t float_end, int rank, int world,
                    void* stream) {
  g_last_error[0] = 0;
  if (!multicast_buffer || world < 1 || rank < 0 || rank >= world || float_begin < 0 || float_end < float_begin ||
      (float_begin & 3) || (float_end & 3))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(multicast_buffer)) return RM_ERR_WORKSPACE;
  if (float_end == float_begin) return RM_OK;
  // a multicast address belongs to no single device: the caller's current device launches
  return rm_launch_multimem_sum(multicast_buffer, float_begin, float_end, rank, world,
                                static_cast<cudaStream_t>(stream));
}

int rm_activate_output(const float* camera_center, const float* density, const float* rgb, const float* grd,
                       const void* sh, int sh_is_half, const int32_t* indices, const float* circumcenters,
                       const float* vertices, int64_t n_tets, int sh_degree, int n_sh_rest, float* features,
                       void* stream) {
  g_last_error[0] = 0;
  if (n_tets < 0 || sh_degree < 0 || sh_degree > 4) return RM_ERR_INVALID_ARG;
  if (n_tets == 0) return RM_OK;
  if (n_sh_rest < (sh_degree + 1) * (sh_degree + 1) - 1 || n_sh_rest > 24) return RM_ERR_INVALID_ARG;
  if (!camera_center || !density || !rgb || !grd || !indices || !circumcenters || !vertices || !features ||
      (sh_degree > 0 && !sh))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(indices)) return RM_ERR_WORKSPACE;
  int rc = rm_bind_device(features);
  if (rc) return rc;
  return rm_launch_activate(camera_center, density, rgb, grd, sh, sh_is_half, indices, circumcenters, vertices,
                            n_tets, sh_degree, n_sh_rest, features, static_cast<cudaStream_t>(stream));
}

int rm_tet_err(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
               const RmCamera* cam, const float* pixel_err, const float* ssim_err, int64_t n_tets, float* tet_err,
               int32_t* tet_count, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || !tile_ranges || !pixel_err || !ssim_err) return RM_ERR_INVALID_ARG;
  if (n_tets == 0) return RM_OK;
  if (!records || !tet_err || !tet_count) return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(records) || !rm_aligned16(tet_err) || (reinterpret_cast<uintptr_t>(tile_ranges) & 7))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(tet_err);
  if (rc) return rc;
  return rm_launch_tet_err(sorted_tetra_idx, tile_ranges, records, cam, pixel_err, ssim_err, n_tets, tet_err,
                           tet_count, static_cast<cudaStream_t>(stream));
}

int rm_vertex_backward(const int32_t* indices, const float* vertices, int64_t n_tets, int64_t n_vertices,
                       const RmCamera* cam, const int32_t* tiles_touched, const float* grad_vs_tetra,
                       const float* grad_circumcenter, float* vertices_grad, void* stream) {
  g_last_error[0] = 0;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0 || !vertices_grad) return RM_ERR_INVALID_ARG;
  if (n_tets > 0 && (!indices || !vertices || !tiles_touched || !grad_vs_tetra || !grad_circumcenter))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(indices)) return RM_ERR_WORKSPACE;
  rc = rm_bind_device(vertices_grad);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RM_CUDA_CHECK(cudaMemsetAsync(vertices_grad, 0, sizeof(float) * 3 * (size_t)n_vertices, st));
  return rm_launch_vertex_backward(indices, vertices, n_tets, cam, tiles_touched, grad_vs_tetra, grad_circumcenter,
                                   vertices_grad, st);
}

}  // extern "C"
