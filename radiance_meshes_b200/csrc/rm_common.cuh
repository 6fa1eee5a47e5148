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

// ---------------------------------------------------------------------------
// Bounds-checked build (-DRM_BOUNDS_CHECK), used by the tests in place of a memory checker: every
// index that depends on data (list cursors, hit-list slots, ids read from lists, rows addressed by
// them) is tested against the extent of its array before the access; a violation sets a bit of a
// status word that rm_debug_bounds_status() returns and the access is skipped - nothing traps.  The
// extents are set by the host launchers before each launch.  In the normal build the macros vanish.
// ---------------------------------------------------------------------------
enum RmExtent {
  RM_X_LIST = 0,      // sorted_tetra_idx entries
  RM_X_TETS,          // records / record-gradient rows / tet_flags / per-tet outputs
  RM_X_VERTS,         // vertices
  RM_X_HIT_IDS,       // hit-list id slots
  RM_X_HIT_MASKS,     // hit-list mask slots
  RM_X_UNITS,         // hit-list counts
  RM_X_PAIRS,         // (region, tet) pairs / sorted region entries
  RM_X_CHUNKS,        // chunks of the level-2 list build
  RM_X_REGIONS,       // regions
  RM_X_TILES,         // tiles
  RM_X_COUNT
};
#ifdef RM_BOUNDS_CHECK
static __device__ long long g_rm_extent[RM_X_COUNT];
static __device__ unsigned g_rm_bounds_status;
// site: a small number naming the access, reported as bit (site & 31)
#define RM_INDEX_OK(i, which, site) rm_index_ok((long long)(i), g_rm_extent[which], (site))
static __device__ __forceinline__ bool rm_index_ok(long long i, long long n, int site) {
  if ((unsigned long long)i < (unsigned long long)n) return true;
  atomicOr(&g_rm_bounds_status, 1u << (site & 31));
  return false;
}
static inline void rm_set_extent(int which, long long n, cudaStream_t st) {
  cudaMemcpyToSymbolAsync(g_rm_extent, &n, sizeof(n), sizeof(long long) * (size_t)which, cudaMemcpyHostToDevice, st);
}
static inline unsigned rm_take_bounds_status() {
  unsigned v = 0, z = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&v, g_rm_bounds_status, sizeof(v));
  cudaMemcpyToSymbol(g_rm_bounds_status, &z, sizeof(z));
  return v;
}
#else
#define RM_INDEX_OK(i, which, site) true
static inline void rm_set_extent(int, long long, cudaStream_t) {}
static inline unsigned rm_take_bounds_status() { return 0; }
#endif
unsigned rm_bounds_status_raster();
unsigned rm_bounds_status_binning();

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
