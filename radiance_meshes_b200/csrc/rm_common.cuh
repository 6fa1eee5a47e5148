// Shared device/host helpers for the sm_100a rasterizer kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "rm_b200.h"

#define RM_CUDA_CHECK(expr)                          \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) {                         \
      rm_set_last_cuda_error(_e, __FILE__, __LINE__); \
      return RM_ERR_CUDA;                            \
    }                                                \
  } while (0)

void rm_set_last_cuda_error(cudaError_t e, const char* file, int line);
void rm_clear_last_error();
int rm_bind_device(const void* device_ptr);
// Host-side checks every entry point applies to its camera and to pointers it accesses with
// 128-bit loads or stores.
int rm_check_cam(const RmCamera* c);
static inline bool rm_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Every kernel launch of the library is counted (rm_launch_count), so that a caller can state how
// many of this library's kernels ran inside a timed region.
void rm_count_launch();

// Optional per-kernel timing (rm_profile_enable): a scope records a CUDA event
// pair on the launch stream around the launches it encloses.
void rm_prof_begin(const char* name, cudaStream_t st);
void rm_prof_end(cudaStream_t st);
struct RmProfScope {
  cudaStream_t st;
  RmProfScope(const char* name, cudaStream_t s) : st(s) { rm_prof_begin(name, s); }
  ~RmProfScope() { rm_prof_end(st); }
};

namespace rm {

constexpr int kRecordFloats = RM_RECORD_FLOATS;

// Camera in registers / shared memory.  Loaded from the device arrays of
// RmCamera so that the host never has to read them back.
struct DevCam {
  float W[16];
  float K[9];
  float pos[3];
  float dist[4];
  int H, Wd, type;
  float min_t;
  int tile_h, tile_w, grid_h, grid_w;
  int row0, row1;
};

__device__ __forceinline__ void load_cam(const RmCamera& c, DevCam& d) {
#pragma unroll
  for (int i = 0; i < 16; ++i) d.W[i] = __ldg(c.world_view_transform + i);
#pragma unroll
  for (int i = 0; i < 9; ++i) d.K[i] = __ldg(c.K + i);
#pragma unroll
  for (int i = 0; i < 3; ++i) d.pos[i] = __ldg(c.cam_pos + i);
#pragma unroll
  for (int i = 0; i < 4; ++i) d.dist[i] = __ldg(c.distortion_params + i);
  d.H = c.image_height;
  d.Wd = c.image_width;
  d.type = c.camera_type;
  d.min_t = c.min_t;
  d.tile_h = c.tile_height;
  d.tile_w = c.tile_width;
  d.grid_h = c.grid_height;
  d.grid_w = c.grid_width;
  d.row0 = c.tile_row_begin;
  d.row1 = c.tile_row_end;
}

struct f3 {
  float x, y, z;
};
__device__ __forceinline__ f3 operator+(f3 a, f3 b) { return {a.x + b.x, a.y + b.y, a.z + b.z}; }
__device__ __forceinline__ f3 operator-(f3 a, f3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
__device__ __forceinline__ f3 operator*(f3 a, float s) { return {a.x * s, a.y * s, a.z * s}; }
__device__ __forceinline__ f3 operator-(f3 a) { return {-a.x, -a.y, -a.z}; }
__device__ __forceinline__ float dot(f3 a, f3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ f3 cross(f3 a, f3 b) {
  return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x};
}
__device__ __forceinline__ f3 load3(const float* p, int64_t i) {
  return {__ldg(p + 3 * i), __ldg(p + 3 * i + 1), __ldg(p + 3 * i + 2)};
}

struct d3 {
  double x, y, z;
};
__device__ __forceinline__ d3 operator+(d3 a, d3 b) { return {a.x + b.x, a.y + b.y, a.z + b.z}; }
__device__ __forceinline__ d3 operator-(d3 a, d3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
__device__ __forceinline__ d3 operator*(d3 a, double s) { return {a.x * s, a.y * s, a.z * s}; }
__device__ __forceinline__ double dot(d3 a, d3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ d3 cross(d3 a, d3 b) {
  return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x};
}

// Order-preserving map float -> uint32 (slang/tile_shader.slang:18-47).
__device__ __forceinline__ uint32_t float2sortable_key(float v) {
  uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
}

}  // namespace rm
