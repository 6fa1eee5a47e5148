// Stages 5-6 on the GPU: per-pixel front-to-back integration of the tile lists
// and its reverse pass.
//
// Reference behaviour reproduced: slang/alphablend_shader_interp.slang:83-431
// (pixel state, distortion moments, forward loop with early termination at
// log-transmittance < -5.5, backward replay with state undo),
// slang/interp_version.slang:21-153 (closed-form segment integral of constant
// density and linear colour), slang/intersect.slang:393-624 (ray/tet slab
// test), slang/camera.slang:241-346 (ray generation).
//
// Design (not the reference's structure):
//   * Tets are packed once per frame into 144-byte records: the four outward
//     face planes relative to the CAMERA POSITION (n_i, D_i), the colour field
//     folded to (grd, s0 = grd.(cam - v0), base, density) - 96 bytes that are
//     staged in shared memory - and the edge lines of the tet's projected hull
//     (48 bytes, read only to decide whether a tet can touch a tile's samples).
//     The per-pixel origin offset o = cam + min_t*d only shifts each plane
//     distance by min_t*(n_i.d), so the per-(pixel,tet) work drops from four
//     cross products to four dot products.
//   * A half-warp owns 16 pixels of one tile; a warp therefore walks two tile
//     lists side by side.  Forward: the list is examined 16 entries at a time
//     (hull lines against the box of the half-warp's samples); survivors are
//     tested against each of the 16 sample positions, which gives the mask of
//     pixels a tet can cover; entries with a non-empty mask are staged 16 at a
//     time with 128-bit cp.async copies, double buffered, and every lane then
//     walks only the staged entries that cover its pixel.  A half-warp stops as
//     soon as all of its pixels have terminated.  Every evaluated batch is
//     appended, with the per-pixel bit sets of the entries that were hit, to the
//     half-warp's hit list.
//   * Backward walks the hit lists back to front, up to three consecutive entries
//     with disjoint pixel masks per step, and accumulates gradients with
//     respect to 16 of the 24 record fields per hit (entering plane, exit plane,
//     colour fields): the 16 pixels' values are summed through a shared-memory
//     transpose when they share both faces, else added with 128-bit atomics, into
//     a per-tet row; a per-tet kernel then applies the chain rule to vertices and
//     cell values (12 vertex atomics per tet instead of 19 atomics per pixel hit).

#include <type_traits>
#include "rm_common.cuh"

namespace rm {

constexpr int kRecStride = RM_RECORD_FLOATS / 4;  // float4 per record in global memory (the first 6 are staged)

// ----------------------------------------------------------------------------
// Record packing
// ----------------------------------------------------------------------------
struct PlaneSetup {
  f3 n[4];
  float D[4];
  float sgn[4];
};

__device__ __forceinline__ void make_planes(const f3 v[4], f3 cam, PlaneSetup& p) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // faces (v0,v1,v2) (v0,v1,v3) (v0,v2,v3) (v1,v2,v3); opposite vertex v3 v2 v1 v0
    const int b = i == 3 ? 1 : 0;
    const int e1 = i < 2 ? 1 : 2;
    const int e2 = i == 0 ? 2 : 3;
    const int op = 3 - i;
    f3 n = cross(v[e1] - v[b], v[e2] - v[b]);
    float s = 1.0f;
    if (dot(n, v[op] - v[b]) > 0.0f) {
      n = -n;
      s = -1.0f;
    }
    p.n[i] = n;
    p.sgn[i] = s;
    p.D[i] = -dot(n, v[b] - cam);
  }
}

constexpr int kPackThreads = 128;

// One thread per tet builds the record in registers; the block then writes its
// records through shared memory so that the global stores are contiguous.
__global__ void __launch_bounds__(kPackThreads, 8)
k_pack_records(const int32_t* __restrict__ indices, const float* __restrict__ vertices,
               const float* __restrict__ cell, int64_t T, int64_t V, RmCamera rcam,
               const int32_t* __restrict__ tiles_touched, float4* __restrict__ records) {
  __shared__ __align__(16) float4 sm[kPackThreads * kRecStride];
  __shared__ bool packed[kPackThreads];  // culled tets appear in no list: their rows are not written
  const int64_t g0 = (int64_t)blockIdx.x * kPackThreads;
  const int64_t g = g0 + threadIdx.x;
  float4 r[kRecStride];
#pragma unroll
  for (int k = 0; k < kRecStride; ++k) r[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool live = g < T && !(tiles_touched && tiles_touched[g] == 0);
  packed[threadIdx.x] = live;
  int4 id = make_int4(0, 0, 0, 0);
  bool ids_ok = false;
  if (live) {
    id = __ldg(reinterpret_cast<const int4*>(indices) + g);
    ids_ok = (uint32_t)id.x < (uint64_t)V && (uint32_t)id.y < (uint64_t)V && (uint32_t)id.z < (uint64_t)V &&
             (uint32_t)id.w < (uint64_t)V;
    // A tet that names a vertex outside the table (the projection stage culls it and reports it) keeps the
    // all-zero planes and gets the always-separating line below: no pixel can hit it.
    if (!ids_ok) r[6] = make_float4(0.0f, 0.0f, -1.0f, 0.0f);
  }
  if (live && ids_ok) {
    f3 cam = {__ldg(rcam.cam_pos), __ldg(rcam.cam_pos + 1), __ldg(rcam.cam_pos + 2)};
    f3 v[4] = {load3(vertices, id.x), load3(vertices, id.y), load3(vertices, id.z), load3(vertices, id.w)};
    PlaneSetup p;
    make_planes(v, cam, p);
    const float* c = cell + 7 * g;
    float density = fmaxf(__ldg(c), 0.0f);
    f3 base = {__ldg(c + 1), __ldg(c + 2), __ldg(c + 3)};
    f3 grd = {__ldg(c + 4), __ldg(c + 5), __ldg(c + 6)};
    float s0 = dot(grd, cam - v[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = make_float4(p.n[i].x, p.n[i].y, p.n[i].z, p.D[i]);
    r[4] = make_float4(grd.x, grd.y, grd.z, s0);
    r[5] = make_float4(base.x, base.y, base.z, density);
    // Vertices in pixel coordinates, for the per-tile cull of the integration
    // kernels.  Only meaningful for an undistorted pinhole with the whole tet in
    // front of the camera; otherwise the cull is disabled for this tet (NaN lines).
    const float* W = rcam.world_view_transform;
    const float* D = rcam.distortion_params;
    const float fx = __ldg(rcam.K + 0), cx = __ldg(rcam.K + 2), fy = __ldg(rcam.K + 4), cy = __ldg(rcam.K + 5);
    const float d2 = __ldg(D) * __ldg(D) + __ldg(D + 1) * __ldg(D + 1) + __ldg(D + 2) * __ldg(D + 2) +
                     __ldg(D + 3) * __ldg(D + 3);
    bool ok = rcam.camera_type == 0 && d2 < 1e-9f;
    float px[4], py[4];
    // Bound of the fp32 rounding error of the projected vertices, in pixels: the camera-space
    // coordinates are sums of four products (error <= 4 * 2^-24 * sum of magnitudes), and the error of
    // X/Z grows with 1/Z, so vertices near the camera plane project with errors far above the 0.01
    // pixel margin of the hull tests.  The lines are moved outwards by the bound (two end points per
    // line); a tet whose bound reaches half a pixel, or with a vertex behind the near plane, is not culled.
    float perr = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float X = __ldg(W + 0) * v[k].x + __ldg(W + 1) * v[k].y + __ldg(W + 2) * v[k].z + __ldg(W + 3);
      float Y = __ldg(W + 4) * v[k].x + __ldg(W + 5) * v[k].y + __ldg(W + 6) * v[k].z + __ldg(W + 7);
      float Z = __ldg(W + 8) * v[k].x + __ldg(W + 9) * v[k].y + __ldg(W + 10) * v[k].z + __ldg(W + 11);
      const float u4 = 2.4e-7f;
      const float eX = u4 * (fabsf(__ldg(W + 0) * v[k].x) + fabsf(__ldg(W + 1) * v[k].y) + fabsf(__ldg(W + 2) * v[k].z) + fabsf(__ldg(W + 3)));
      const float eY = u4 * (fabsf(__ldg(W + 4) * v[k].x) + fabsf(__ldg(W + 5) * v[k].y) + fabsf(__ldg(W + 6) * v[k].z) + fabsf(__ldg(W + 7)));
      const float eZ = u4 * (fabsf(__ldg(W + 8) * v[k].x) + fabsf(__ldg(W + 9) * v[k].y) + fabsf(__ldg(W + 10) * v[k].z) + fabsf(__ldg(W + 11)));
      ok = ok && Z > 1e-3f;
      const float iz = 1.0f / Z;
      px[k] = fx * (X / Z) + cx;
      py[k] = fy * (Y / Z) + cy;
      const float ex = fabsf(fx) * iz * (eX + fabsf(X * iz) * eZ) + 4e-7f * (fabsf(px[k]) + fabsf(cx));
      const float ey = fabsf(fy) * iz * (eY + fabsf(Y * iz) * eZ) + 4e-7f * (fabsf(py[k]) + fabsf(cy));
      perr = fmaxf(perr, ex + ey);
    }
    const float margin = 2.0f * perr;
    ok = ok && margin < 0.5f;
    // Edge lines of the convex hull of the four projected vertices, a*x + b*y + c >= 0
    // inside, (a, b) of unit length.  A vertex pair is a hull edge iff the other two
    // vertices lie on one side of its line; a tet projects to a quadrilateral (4 such
    // pairs) or to a triangle with one vertex inside (3).  Anything else is degenerate
    // and disables the cull for this tet.
    float la[4] = {0, 0, 0, 0}, lb[4] = {0, 0, 0, 0}, lc[4] = {0, 0, 0, 0};
    int ne = 0;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
      for (int b = a + 1; b < 4; ++b) {
        const int c1 = (a != 0 && b != 0) ? 0 : ((a != 1 && b != 1) ? 1 : 2);
        const int c2 = 6 - a - b - c1;
        float nx = -(py[b] - py[a]), ny = px[b] - px[a];
        const float len = sqrtf(nx * nx + ny * ny);
        const float s1 = nx * (px[c1] - px[a]) + ny * (py[c1] - py[a]);
        const float s2 = nx * (px[c2] - px[a]) + ny * (py[c2] - py[a]);
        const bool pos = s1 >= 0.0f && s2 >= 0.0f && (s1 > 0.0f || s2 > 0.0f);
        const bool neg = s1 <= 0.0f && s2 <= 0.0f && (s1 < 0.0f || s2 < 0.0f);
        if ((pos || neg) && len > 0.0f) {
          const float inv = (pos ? 1.0f : -1.0f) / len;
          nx *= inv;
          ny *= inv;
          const float cc = -(nx * px[a] + ny * py[a]) + margin;
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // slot `ne`, without dynamic indexing
            if (q == ne) { la[q] = nx; lb[q] = ny; lc[q] = cc; }
          }
          ++ne;
        }
      }
    }
    ok = ok && (ne == 3 || ne == 4);
    if (ne == 3) { la[3] = la[2]; lb[3] = lb[2]; lc[3] = lc[2]; }
    const float qnan = __int_as_float(0x7fc00000);
    if (!ok) {
#pragma unroll
      for (int k = 0; k < 4; ++k) la[k] = lb[k] = lc[k] = qnan;
    }
    // A tet of zero density can neither contribute nor terminate a pixel: its first line separates
    // every sample box, so the examination of the integration kernels drops it without reading more.
    if (!(density > 0.0f)) { la[0] = 0.0f; lb[0] = 0.0f; lc[0] = -1.0f; }
    r[6] = make_float4(la[0], lb[0], lc[0], la[1]);
    r[7] = make_float4(lb[1], lc[1], la[2], lb[2]);
    r[8] = make_float4(lc[2], la[3], lb[3], lc[3]);
  }
#pragma unroll
  for (int k = 0; k < kRecStride; ++k) sm[threadIdx.x * kRecStride + k] = r[k];
  __syncthreads();
  const int64_t n_rec = min((int64_t)kPackThreads, T - g0);
  float4* out = records + g0 * kRecStride;
  for (int i = threadIdx.x; i < n_rec * kRecStride; i += kPackThreads)
    if (packed[i / kRecStride]) out[i] = sm[i];
}

// True if one of the four hull edge lines of a tet's projection (l0, l1, l2) has the
// whole box [X0,X1] x [Y0,Y1] of a half-warp's sample positions on its outer side
// by more than 0.01 pixel.  Conservative: NaN lines never separate.
__device__ __forceinline__ bool hull_misses_box(float4 l0, float4 l1, float4 l2, float X0, float X1, float Y0,
                                                float Y1) {
  const float a[4] = {l0.x, l0.w, l1.z, l2.y};
  const float b[4] = {l0.y, l1.x, l1.w, l2.z};
  const float c[4] = {l0.z, l1.y, l2.x, l2.w};
  bool sep = false;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float hi = fmaf(a[k], a[k] > 0.0f ? X1 : X0, fmaf(b[k], b[k] > 0.0f ? Y1 : Y0, c[k]));
    sep = sep || hi < -0.01f;
  }
  return sep;
}

// ----------------------------------------------------------------------------
// Ray generation (fp32), slang/camera.slang:241-346
// ----------------------------------------------------------------------------
__device__ __forceinline__ void undistort(float& px, float& py, const float* dist) {
  float k1 = dist[0], k2 = dist[1], p1 = dist[2], p2 = dist[3];
  if (k1 * k1 + k2 * k2 + p1 * p1 + p2 * p2 < 1e-9f) return;
  float x = px, y = py;
  for (int i = 0; i < 10; ++i) {
    float r2 = x * x + y * y;
    float d = 1.0f + r2 * (k1 + r2 * k2);
    float fx = d * x + 2.0f * p1 * x * y + p2 * (r2 + 2.0f * x * x) - px;
    float fy = d * y + 2.0f * p2 * x * y + p1 * (r2 + 2.0f * y * y) - py;
    float d_r = k1 + r2 * (2.0f * k2);
    float d_x = 2.0f * x * d_r;
    float d_y = 2.0f * y * d_r;
    float fx_x = d + d_x * x + 2.0f * p1 * y + 6.0f * p2 * x;
    float fx_y = d_y * x + 2.0f * p1 * x + 2.0f * p2 * y;
    float fy_x = d_x * y + 2.0f * p2 * y + 2.0f * p1 * x;
    float fy_y = d + d_y * y + 2.0f * p2 * x + 6.0f * p1 * y;
    float denom = fy_x * fx_y - fx_x * fy_y;
    if (fabsf(denom) < 1e-9f) break;
    float xn = fx * fy_y - fy * fx_y;
    float yn = fy * fx_x - fx * fy_x;
    x += xn / denom;
    y += yn / denom;
  }
  px = x;
  py = y;
}

__device__ __forceinline__ f3 ray_direction(const RmCamera& c, float px, float py) {
  float fx = __ldg(c.K + 0), cx = __ldg(c.K + 2), fy = __ldg(c.K + 4), cy = __ldg(c.K + 5);
  float x = (px - cx) / fx, y = (py - cy) / fy;
  float dist[4] = {__ldg(c.distortion_params), __ldg(c.distortion_params + 1), __ldg(c.distortion_params + 2),
                   __ldg(c.distortion_params + 3)};
  if (c.camera_type == 0 || c.camera_type == 1) undistort(x, y, dist);
  f3 dc;
  if (c.camera_type == 1) {
    float theta = sqrtf(x * x + y * y);
    theta = fminf(3.14159265f, theta);
    float s = (theta < 1e-6f) ? 1.0f : sinf(theta) / theta;
    dc = {x * s, y * s, cosf(theta)};
  } else {
    float l = sqrtf(x * x + y * y + 1.0f);
    dc = {x / l, y / l, 1.0f / l};
  }
  const float* W = c.world_view_transform;
  f3 w = {__ldg(W + 0) * dc.x + __ldg(W + 4) * dc.y + __ldg(W + 8) * dc.z,
          __ldg(W + 1) * dc.x + __ldg(W + 5) * dc.y + __ldg(W + 9) * dc.z,
          __ldg(W + 2) * dc.x + __ldg(W + 6) * dc.y + __ldg(W + 10) * dc.z};
  float l = sqrtf(dot(w, w));
  return {w.x / l, w.y / l, w.z / l};
}

// ----------------------------------------------------------------------------
// Per (pixel, record) evaluation shared by forward and backward
// ----------------------------------------------------------------------------
struct Eval {
  float enter, exit, te, tx;  // clamped and raw distances (from the offset origin)
  int ie, ix;                 // planes that produced te / tx (-1: none)
  float dt, tau, gd, oe, ox, alpha, phi, w0, w1;
  float cr, cg, cb;           // colour contribution
};

// The entering and exit distances are plain max/min chains over the four planes:
// a plane the ray crosses inwards (den < 0) bounds the entry, one it crosses outwards
// (den > 0) the exit.  The reference ignores a plane with |den| < 1e-10 unless the
// origin lies outside it, which is a miss (slang/intersect.slang:478-607).  The chains
// give the same answers without the special case: such a plane's distance -D/den is
// huge, positive when the origin is outside (the entry passes the exit: a miss) and
// negative when it is inside (no effect on the maximum), and symmetrically for the
// exit.  A denominator of exactly zero gives +-inf with the sign that rejects the ray
// when the origin is outside and changes nothing when it is inside, provided -0 counts
// as "crossing inwards": the direction of a plane is therefore read from the sign bit
// of den, not from den < 0.  0/0 is NaN, which fmaxf/fminf drop (the reference ignores
// that plane too).
// TRACK = true (backward) also reports which plane produced each distance: the first
// plane, in index order, whose distance equals the chain's result.  It runs the chains
// as "strictly greater / strictly smaller" updates that carry the index along; these
// leave the same values as fmaxf/fminf (a NaN never compares greater or smaller).
template <bool TRACK>
__device__ __forceinline__ bool slab_test(const float4 (&rec)[4], f3 d, float min_t, Eval& e) {
  // Distances are first taken from the camera position (u = -D/den) and shifted
  // by min_t afterwards: t = -(D + min_t*den)/den = u - min_t.
  float ue = -1e30f, ux = 1e30f;
  int ie = -1, ix = -1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 p = rec[i];
    const float den = p.x * d.x + p.y * d.y + p.z * d.z;
    const float u = __fdividef(-p.w, den);
    const bool ent = __float_as_int(den) < 0;  // sign bit: -0 bounds the entry, +0 the exit
    if (TRACK) {
      const bool later = ent && u > ue, sooner = !ent && u < ux;
      ue = later ? u : ue;
      ie = later ? i : ie;
      ux = sooner ? u : ux;
      ix = sooner ? i : ix;
    } else {
      ue = fmaxf(ue, ent ? u : -1e30f);
      ux = fminf(ux, ent ? 1e30f : u);
    }
  }
  const float te = ue - min_t, tx = ux - min_t;
  if (!(te <= tx) || tx <= 0.0f) return false;
  e.te = te; e.tx = tx; e.ie = ie; e.ix = ix;
  e.enter = fmaxf(te, 0.0f);
  e.exit = fmaxf(tx, e.enter);
  e.dt = fmaxf(e.exit - e.enter, 0.0f);
  return true;
}

// Weights of the closed-form segment integral for optical depth x > 0:
//   alpha = exp(-x), phi = (1 - alpha)/x, w0 = phi - alpha, w1 = 1 - phi.
// Below x = 0.25 the differences cancel, so w0 and w1 come from their Taylor
// series (truncation < 1e-7 relative); above, from the fast exponential.
__device__ __forceinline__ void segment_weights(float x, float& alpha, float& phi, float& w0, float& w1) {
  alpha = __expf(-x);
  if (x < 0.25f) {
    // w1 = x/2 - x^2/6 + x^3/24 - x^4/120 + x^5/720 - x^6/5040
    w1 = x * fmaf(x, fmaf(x, fmaf(x, fmaf(x, fmaf(x, -1.0f / 5040.0f, 1.0f / 720.0f), -1.0f / 120.0f), 1.0f / 24.0f),
                          -1.0f / 6.0f), 0.5f);
    // w0 = x/2 - x^2/3 + x^3/8 - x^4/30 + x^5/144 - x^6/840
    w0 = x * fmaf(x, fmaf(x, fmaf(x, fmaf(x, fmaf(x, -1.0f / 840.0f, 1.0f / 144.0f), -1.0f / 30.0f), 0.125f),
                          -1.0f / 3.0f), 0.5f);
    phi = 1.0f - w1;
  } else {
    phi = __fdividef(1.0f - alpha, x);
    w0 = phi - alpha;
    w1 = 1.0f - phi;
  }
}

// returns false if the segment contributes nothing (optical depth not > 0)
__device__ __forceinline__ bool integrate(const float4* __restrict__ rec, f3 d, float min_t, Eval& e) {
  float4 cg = rec[4], cb = rec[5];
  e.tau = cb.w * e.dt;
  if (!(e.tau > 0.0f)) return false;
  e.gd = cg.x * d.x + cg.y * d.y + cg.z * d.z;
  e.oe = fmaf(e.enter + min_t, e.gd, cg.w);
  e.ox = fmaf(e.exit + min_t, e.gd, cg.w);
  segment_weights(e.tau, e.alpha, e.phi, e.w0, e.w1);
  e.cr = e.w0 * (cb.x + e.ox) + e.w1 * (cb.x + e.oe);
  e.cg = e.w0 * (cb.y + e.ox) + e.w1 * (cb.y + e.oe);
  e.cb = e.w0 * (cb.z + e.ox) + e.w1 * (cb.z + e.oe);
  return true;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
// The hull edge lines of a record (bytes 96..143) are wanted soon: start their way into the caches.
__device__ __forceinline__ void prefetch_hull_lines(const float4* rec) {
  asm volatile("prefetch.global.L1 [%0];\n" ::"l"(rec + 6));
  asm volatile("prefetch.global.L1 [%0];\n" ::"l"(rec + 8));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

constexpr int kWarpsPerBlock = 4;
constexpr int kChunk = 16;  // records staged per half-warp per round
constexpr int kBwdGroup = 3;        // entries with disjoint pixel masks the backward walk takes in one step
constexpr int kTileSumMinHits = 4;  // fewer hit pixels in a tile: every pixel adds its own values with atomics

struct Unit {
  int tile;       // linear tile index
  int x, y;       // pixel
  bool inside;    // pixel exists
  int start, len; // tile list
  int sub, subs;  // which 16-pixel group of the tile this half-warp owns, out of how many
};

__device__ __forceinline__ Unit make_unit(const RmCamera& c, const int2* __restrict__ ranges, int64_t unit,
                                          int64_t n_units, int subs, int lane16) {
  Unit u;
  u.inside = false;
  u.start = 0;
  u.len = 0;
  u.tile = 0;
  u.x = u.y = 0;
  u.sub = 0;
  u.subs = subs;
  if (unit >= n_units) return u;
  int64_t t = unit / subs;
  int sub = (int)(unit - t * subs);
  u.tile = c.tile_row_begin * c.grid_width + (int)t;
  int ty = u.tile / c.grid_width, tx = u.tile - ty * c.grid_width;
  u.sub = sub;
  int p = sub * 16 + lane16;
  int ly = p / c.tile_width, lx = p - ly * c.tile_width;
  u.x = tx * c.tile_width + lx;
  u.y = ty * c.tile_height + ly;
  u.inside = ly < c.tile_height && u.x < c.image_width && u.y < c.image_height;
  int2 rg = __ldg(ranges + u.tile);
  u.start = rg.x;
  u.len = rg.y - rg.x;
  if (u.len > 0 && !(RM_INDEX_OK(rg.x, RM_X_LIST, 0) && RM_INDEX_OK(rg.y - 1, RM_X_LIST, 0))) u.len = 0;
  return u;
}

// Bounding box of the sample positions (pixel + jitter) of the half-warp's pixels.
__device__ __forceinline__ void halfwarp_sample_box(bool inside, float sx, float sy, float& X0, float& X1, float& Y0,
                                                    float& Y1) {
  X0 = inside ? sx : 3.0e38f;
  X1 = inside ? sx : -3.0e38f;
  Y0 = inside ? sy : 3.0e38f;
  Y1 = inside ? sy : -3.0e38f;
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) {
    X0 = fminf(X0, __shfl_xor_sync(0xffffffffu, X0, o));
    X1 = fmaxf(X1, __shfl_xor_sync(0xffffffffu, X1, o));
    Y0 = fminf(Y0, __shfl_xor_sync(0xffffffffu, Y0, o));
    Y1 = fmaxf(Y1, __shfl_xor_sync(0xffffffffu, Y1, o));
  }
}

// ----------------------------------------------------------------------------
// Forward
// ----------------------------------------------------------------------------
// A half-warp owns 16 pixels of one tile and walks the tile's list in three stages that
// are decoupled by two small queues in shared memory (ring buffers of 32 slots):
//   1. examination, 16 entries at a time: every lane reads the hull lines of one entry
//      (48 bytes, prefetched one chunk ahead) and tests them against the bounding box of
//      the half-warp's sample positions (zero density is encoded as an always-separating
//      line by k_pack_records); survivors go to queue A in list order with their position;
//   2. when both half-warps hold 16 entries in queue A (or have nothing left to examine),
//      every lane takes one of them and tests the hull lines against each of the 16 sample
//      positions, which gives the mask of the pixels whose ray can touch the tet; entries
//      with an empty mask are dropped, the others go to queue B with their mask;
//   3. when both half-warps hold 16 entries in queue B (or have run dry), their records
//      (96 bytes each) are staged with 128-bit cp.async, double buffered, and the batch
//      staged one round earlier is evaluated: the masks are transposed so that every
//      lane (= pixel) holds the bit set of the batch entries that cover it, and every
//      lane walks its own bits in list order.  Lanes therefore work on different entries
//      at the same time and no lane runs a slab test for a tet that cannot cover its
//      pixel.  A pixel stops at its termination threshold; a half-warp stops examining
//      once all of its pixels have stopped.
// For the backward pass every evaluated batch is appended to the half-warp's hit list:
// the tet ids of the batch and, per pixel, the bit set of the batch entries it hit.
constexpr int kBatch = 16;       // entries staged and evaluated per half-warp and round
constexpr int kRing = 32;        // slots of each candidate queue
constexpr int kStageStride = 7;  // float4 per staged record: 6 used; the odd stride spreads the records over the banks

// The Tukey power ladder of the constant-colour variant (slang/alphablend_shader.slang:26-33):
// sign(x) |p-1|/p ((|x|/|p-1| + 1)^p - 1).
__device__ __forceinline__ float tukey_power_ladder(float x, float p) {
  const float q = fmaxf(fabsf(p - 1.0f), 1.0754944e-20f);
  const float y = fabsf(p - 1.0f) / p * (__powf(fabsf(x) / q + 1.0f, p) - 1.0f);
  return x > 0.0f ? y : (x < 0.0f ? -y : 0.0f);
}

// Mask of the sample positions sp[0..15] that lie inside (or within 0.01 pixel of) the convex hull
// given by four edge lines; NaN lines (cull disabled for the tet) give the full mask.
__device__ __forceinline__ uint32_t hull_pixel_mask(float4 l0, float4 l1, float4 l2, const float2* __restrict__ sp) {
  const float a0 = l0.x, b0 = l0.y, c0 = l0.z + 0.01f;
  const float a1 = l0.w, b1 = l1.x, c1 = l1.y + 0.01f;
  const float a2 = l1.z, b2 = l1.w, c2 = l2.x + 0.01f;
  const float a3 = l2.y, b3 = l2.z, c3 = l2.w + 0.01f;
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float4 s = *reinterpret_cast<const float4*>(sp + i);  // two sample positions
    const float e0 = fminf(fminf(fmaf(a0, s.x, fmaf(b0, s.y, c0)), fmaf(a1, s.x, fmaf(b1, s.y, c1))),
                           fminf(fmaf(a2, s.x, fmaf(b2, s.y, c2)), fmaf(a3, s.x, fmaf(b3, s.y, c3))));
    const float e1 = fminf(fminf(fmaf(a0, s.z, fmaf(b0, s.w, c0)), fmaf(a1, s.z, fmaf(b1, s.w, c1))),
                           fminf(fmaf(a2, s.z, fmaf(b2, s.w, c2)), fmaf(a3, s.z, fmaf(b3, s.w, c3))));
    if (!(e0 < 0.0f)) m |= 1u << i;
    if (!(e1 < 0.0f)) m |= 2u << i;
  }
  return m;
}

// Bit j of the result = bit `lane16` of word j of the 16 masks at `masks` (16-byte aligned).
__device__ __forceinline__ uint32_t transpose_masks(const uint32_t* __restrict__ masks, int lane16) {
  uint32_t bits = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 w = reinterpret_cast<const uint4*>(masks)[q];
    bits |= ((w.x >> lane16) & 1u) << (4 * q);
    bits |= ((w.y >> lane16) & 1u) << (4 * q + 1);
    bits |= ((w.z >> lane16) & 1u) << (4 * q + 2);
    bits |= ((w.w >> lane16) & 1u) << (4 * q + 3);
  }
  return bits;
}

// CONST_COLOR = false: the interpolated-colour renderer (slang/alphablend_shader_interp.slang).
// CONST_COLOR = true: the constant-colour debug renderer (slang/alphablend_shader.slang:100-182,
// utils.slang:160-186): records packed with a zero colour gradient, samples at the pixel centres
// (jitter == nullptr), pixel state (rgb, transmittance) with alpha = 1 - exp(-density * dt), four
// distortion moments weighted by transmittance * alpha with the power ladder of the entry distance,
// termination when the transmittance falls below 1/255; out_img = (r, g, b, transmittance) and
// dist_img has four channels.
template <bool CONST_COLOR>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 5)
k_forward(const int32_t* __restrict__ list, const int2* __restrict__ ranges, const float4* __restrict__ records,
          RmCamera rcam, const float2* __restrict__ jitter, float4* __restrict__ out_img,
          float* __restrict__ dist_img, int32_t* __restrict__ n_contrib, int32_t* __restrict__ hit_counts,
          int32_t* __restrict__ hit_ids, uint16_t* __restrict__ hit_masks, uint8_t* __restrict__ tet_flags,
          int subs, int64_t n_units, float pre_multi, float ladder_p) {
  __shared__ __align__(16) float4 stage[kWarpsPerBlock][2][2][kBatch * kStageStride];  // [warp][half][buffer]
  __shared__ __align__(16) float2 samples[kWarpsPerBlock][2][16];
  __shared__ int qa_id[kWarpsPerBlock][2][kRing], qa_pos[kWarpsPerBlock][2][kRing];
  __shared__ int qb_id[kWarpsPerBlock][2][kRing], qb_pos[kWarpsPerBlock][2][kRing];
  __shared__ uint32_t qb_mask[kWarpsPerBlock][2][kRing];
  __shared__ int batch_id[kWarpsPerBlock][2][2][kBatch], batch_pos[kWarpsPerBlock][2][2][kBatch];
  __shared__ __align__(16) uint32_t batch_mask[kWarpsPerBlock][2][2][kBatch];
  constexpr unsigned FULL = 0xffffffffu;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, lane16 = lane & 15;
  const unsigned below = (1u << lane16) - 1u;
  const int64_t unit = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * 2 + half;
  Unit u = make_unit(rcam, ranges, unit, n_units, subs, lane16);
  int* a_id = qa_id[warp][half];
  int* a_pos = qa_pos[warp][half];
  int* b_id = qb_id[warp][half];
  int* b_pos = qb_pos[warp][half];
  uint32_t* b_mask = qb_mask[warp][half];

  f3 d = {0.f, 0.f, 1.f};
  const int64_t pix = (int64_t)u.y * rcam.image_width + u.x;
  float sx = 0.f, sy = 0.f;
  if (u.inside) {
    float2 j = jitter ? __ldg(jitter + pix) : make_float2(0.5f, 0.5f);
    sx = (float)u.x + j.x;
    sy = (float)u.y + j.y;
    d = ray_direction(rcam, sx, sy);
  }
  samples[warp][half][lane16] = make_float2(sx, sy);
  const float min_t = rcam.min_t;
  float X0, X1, Y0, Y1;
  halfwarp_sample_box(u.inside, sx, sy, X0, X1, Y0, Y1);

  float sr = 0.f, sg = 0.f, sb = 0.f, logT = 0.f, T = 1.f;
  float dx = 0.f, dy = 0.f, dz = 0.f, dw = 0.f, dv = 0.f;
  int contrib = 0;
  bool active = u.inside;
  unsigned act16 = (__ballot_sync(FULL, active) >> (16 * half)) & 0xFFFFu;  // pixels of this half still walking
  bool fetching = act16 != 0;

  // Hit list of this half-warp: the tet ids of every evaluated batch at [hbase, hbase + n_ent), and for
  // batch b the 16 per-pixel bit sets at [mbase + 16 b, + 16).  Every batch but the last holds 16 entries.
  const int64_t hbase = (int64_t)u.start * u.subs + (int64_t)u.sub * u.len;
  const int64_t mbase = hbase + 16 * ((int64_t)u.tile * u.subs + u.sub);
  int n_ent = 0;

  // examination state: entry src + lane16 is the one this lane examines next; its tet id and hull
  // lines are already in registers, the id of the entry after it is in flight
  int src = 0;
  int qa_h = 0, qa_n = 0, qb_h = 0, qb_n = 0;  // ring heads and fill levels (the same in all lanes of the half)
  int id_e = (fetching && lane16 < u.len) ? __ldg(list + u.start + lane16) : -1;
  int id_n = (fetching && kBatch + lane16 < u.len) ? __ldg(list + u.start + kBatch + lane16) : -1;
  if (id_e >= 0 && !RM_INDEX_OK(id_e, RM_X_TETS, 1)) id_e = -1;
  if (id_n >= 0 && !RM_INDEX_OK(id_n, RM_X_TETS, 1)) id_n = -1;
  int id_n2 = (fetching && 2 * kBatch + lane16 < u.len) ? __ldg(list + u.start + 2 * kBatch + lane16) : -1;
  if (id_n2 >= 0 && !RM_INDEX_OK(id_n2, RM_X_TETS, 1)) id_n2 = -1;
  if (id_n >= 0) prefetch_hull_lines(records + kRecStride * (int64_t)id_n);
  const float qnan = __int_as_float(0x7fc00000);
  float4 hq0 = make_float4(qnan, qnan, qnan, qnan), hq1 = hq0, hq2 = hq0;
  if (id_e >= 0) {
    const float4* src_rec = records + kRecStride * (int64_t)id_e;
    hq0 = __ldg(src_rec + 6);
    hq1 = __ldg(src_rec + 7);
    hq2 = __ldg(src_rec + 8);
  }

  int buf = 0;    // buffer holding the batch to evaluate
  int n_cur = 0;  // its number of entries
  __syncwarp();
  for (;;) {
    {
      const bool done = !fetching || (n_cur == 0 && qb_n == 0 && qa_n == 0 && src >= u.len);
      if (__all_sync(FULL, done)) break;
    }
    // ---- stages 1 and 2: until both halves hold a full batch in queue B or have run dry
    for (;;) {
      const bool need_b = fetching && qb_n < kBatch && (qa_n > 0 || src < u.len);
      if (!__any_sync(FULL, need_b)) break;
      const bool ready_a = !need_b || qa_n >= kBatch || src >= u.len;
      if (!__all_sync(FULL, ready_a)) {
        const bool ex = need_b && !ready_a;
        const bool cand = ex && id_e >= 0 && !hull_misses_box(hq0, hq1, hq2, X0, X1, Y0, Y1);
        const unsigned cb = (__ballot_sync(FULL, cand) >> (16 * half)) & 0xFFFFu;
        if (cand) {
          const int slot = (qa_h + qa_n + __popc(cb & below)) & (kRing - 1);
          a_id[slot] = id_e;
          a_pos[slot] = src + lane16;
        }
        if (ex) {
          qa_n += __popc(cb);
          src += kBatch;
          id_e = id_n;
          if (id_e >= 0) {
            const float4* src_rec = records + kRecStride * (int64_t)id_e;
            hq0 = __ldg(src_rec + 6);
            hq1 = __ldg(src_rec + 7);
            hq2 = __ldg(src_rec + 8);
          }
          // the id two batches ahead arrived a step ago: its hull lines are asked for now and read in the next step
          id_n = id_n2;
          if (id_n >= 0) prefetch_hull_lines(records + kRecStride * (int64_t)id_n);
          id_n2 = (src + 2 * kBatch + lane16 < u.len) ? __ldg(list + u.start + src + 2 * kBatch + lane16) : -1;
          if (id_n2 >= 0 && !RM_INDEX_OK(id_n2, RM_X_TETS, 1)) id_n2 = -1;
        }
        continue;
      }
      __syncwarp();
      const int take_a = need_b ? min(qa_n, kBatch) : 0;
      uint32_t m = 0;
      int cid = 0, cpos = 0;
      if (lane16 < take_a) {
        const int slot = (qa_h + lane16) & (kRing - 1);
        cid = a_id[slot];
        cpos = a_pos[slot];
        const float4* src_rec = records + kRecStride * (int64_t)cid;
        m = hull_pixel_mask(__ldg(src_rec + 6), __ldg(src_rec + 7), __ldg(src_rec + 8), samples[warp][half]) & act16;
      }
      const unsigned lb = (__ballot_sync(FULL, m != 0u) >> (16 * half)) & 0xFFFFu;
      if (m) {
        const int slot = (qb_h + qb_n + __popc(lb & below)) & (kRing - 1);
        b_id[slot] = cid;
        b_pos[slot] = cpos;
        b_mask[slot] = m;
      }
      qa_h = (qa_h + take_a) & (kRing - 1);
      qa_n -= take_a;
      qb_n += __popc(lb);
      __syncwarp();
    }
    __syncwarp();
    // ---- stage 3a: stage the next batch, the first min(qb_n, 16) entries of queue B
    const int nb = buf ^ 1;
    const int take = fetching ? min(qb_n, kBatch) : 0;
    if (lane16 < take) {
      const int slot = (qb_h + lane16) & (kRing - 1);
      const int id = b_id[slot];
      batch_id[warp][half][nb][lane16] = id;
      batch_pos[warp][half][nb][lane16] = b_pos[slot];
      batch_mask[warp][half][nb][lane16] = b_mask[slot];
      const float4* src_rec = records + kRecStride * (int64_t)id;
      float4* dst = stage[warp][half][nb] + lane16 * kStageStride;
#pragma unroll
      for (int k = 0; k < 6; ++k) cp_async16(dst + k, src_rec + k);
    } else {
      batch_mask[warp][half][nb][lane16] = 0u;
    }
    cp_async_commit();
    qb_h = (qb_h + take) & (kRing - 1);
    qb_n -= take;
    cp_async_wait<1>();
    __syncwarp();
    // ---- stage 3b: evaluate the batch staged one round ago; every lane walks the entries covering its pixel
    const float4* cur = stage[warp][half][buf];
    const int* cur_pos = batch_pos[warp][half][buf];
    uint32_t bits = (active && n_cur > 0) ? transpose_masks(batch_mask[warp][half][buf], lane16) : 0u;
    uint32_t hitbits = 0;
    while (bits) {
      const int j = __ffs(bits) - 1;
      bits &= bits - 1;
      const float4* rec = cur + j * kStageStride;
      const float4 pl[4] = {rec[0], rec[1], rec[2], rec[3]};
      Eval e;
      if (slab_test<false>(pl, d, min_t, e) && integrate(rec, d, min_t, e)) {
        hitbits |= 1u << j;
        sr = fmaf(e.cr, T, sr);
        sg = fmaf(e.cg, T, sg);
        sb = fmaf(e.cb, T, sb);
        bool finished;
        if (CONST_COLOR) {
          const float weight = T * (1.0f - e.alpha);
          const float mm = tukey_power_ladder(e.enter * pre_multi, ladder_p);
          dx = fmaf(2.0f * weight * mm, dz, dx);
          dy = fmaf(2.0f * weight, dw, dy);
          dz += weight;
          dw = fmaf(weight, mm, dw);
          T *= e.alpha;
          finished = T < 1.0f / 255.0f;
        } else {
          logT -= e.tau;
          T *= e.alpha;
          const float dens = rec[5].w;
          const float m1 = dens * (e.exit + e.enter) * 0.5f;
          dx = fmaf(2.0f * m1, dz, dx);
          dy = fmaf(2.0f * dens, dw, dy);
          dz += dens;
          dw += m1;
          dv = fmaf(dens * dens, e.dt * (1.0f / 3.0f), dv);
          finished = logT < -5.5f;
        }
        if (finished) {
          active = false;
          contrib = cur_pos[j] + 1;  // entries walked, the terminating one included
          bits = 0;
        }
      }
    }
    __syncwarp();
    if (hit_ids && n_cur > 0) {  // append the batch to the hit list
      if (lane16 < n_cur && RM_INDEX_OK(hbase + n_ent + lane16, RM_X_HIT_IDS, 2)) {
        const int id = batch_id[warp][half][buf][lane16];
        hit_ids[hbase + n_ent + lane16] = id;
        tet_flags[id] = 1;  // this tet's record-gradient row is cleared and read by the backward pass
      }
      if (RM_INDEX_OK(mbase + n_ent + lane16, RM_X_HIT_MASKS, 3))
        hit_masks[mbase + n_ent + lane16] = (uint16_t)hitbits;  // n_ent is a multiple of 16 here
      n_ent += n_cur;
    }
    act16 = (__ballot_sync(FULL, active) >> (16 * half)) & 0xFFFFu;
    fetching = act16 != 0;
    buf = nb;
    n_cur = take;
  }
  cp_async_wait<0>();
  if (active) contrib = u.len;  // walked the whole list

  if (hit_counts && lane16 == 0 && unit < n_units && RM_INDEX_OK((int64_t)u.tile * u.subs + u.sub, RM_X_UNITS, 4))
    hit_counts[(int64_t)u.tile * u.subs + u.sub] = n_ent;
  if (u.inside) {
    if (CONST_COLOR) {
      out_img[pix] = make_float4(sr, sg, sb, T);
      reinterpret_cast<float4*>(dist_img)[pix] = make_float4(dx, dy, dz, dw);
    } else {
      out_img[pix] = make_float4(sr, sg, sb, logT);
      float* o = dist_img + 5 * pix;
      o[0] = dx; o[1] = dy; o[2] = dz; o[3] = dw; o[4] = dv;
    }
    n_contrib[pix] = contrib;
  }
}

// ----------------------------------------------------------------------------
// Backward
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 5)
k_backward(const int2* __restrict__ ranges, const float4* __restrict__ records, RmCamera rcam,
           const float2* __restrict__ jitter, const float4* __restrict__ out_img, const float* __restrict__ dist_img,
           const int32_t* __restrict__ hit_counts, const int32_t* __restrict__ hit_ids,
           const uint16_t* __restrict__ hit_masks, const float4* __restrict__ g_img, const float* __restrict__ g_dist,
           float* __restrict__ grec, int subs, int64_t n_units) {
  __shared__ __align__(16) float4 stage[kWarpsPerBlock][2][2][kChunk * 6];
  __shared__ int stage_id[kWarpsPerBlock][2][2][kChunk];
  __shared__ unsigned stage_mask[kWarpsPerBlock][2][2][kChunk];  // pixels of the tile that hit the entry (forward)
  __shared__ __align__(16) float reduce_buf[kWarpsPerBlock][2 * (kChunk * 20 + 16)];
  __shared__ __align__(16) uint32_t lane_bits[kWarpsPerBlock][2][kChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, lane16 = lane & 15;
  const int64_t unit = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * 2 + half;
  Unit u = make_unit(rcam, ranges, unit, n_units, subs, lane16);

  f3 d = {0.f, 0.f, 1.f};
  const int64_t pix = (int64_t)u.y * rcam.image_width + u.x;
  float logT = 0.f, sz = 0.f, sw = 0.f;
  float gr = 0.f, gg = 0.f, gb = 0.f, glogT = 0.f, gx = 0.f, gy = 0.f, gz = 0.f, gw = 0.f, gv = 0.f;
  if (u.inside) {
    float2 j = __ldg(jitter + pix);
    d = ray_direction(rcam, (float)u.x + j.x, (float)u.y + j.y);
    logT = __ldg(out_img + pix).w;
    sz = __ldg(dist_img + 5 * pix + 2);
    sw = __ldg(dist_img + 5 * pix + 3);
    float4 g4 = __ldg(g_img + pix);
    gr = g4.x; gg = g4.y; gb = g4.z; glogT = g4.w;
    const float* gd = g_dist + 5 * pix;
    gx = __ldg(gd); gy = __ldg(gd + 1); gz = __ldg(gd + 2); gw = __ldg(gd + 3); gv = __ldg(gd + 4);
  }
  const float min_t = rcam.min_t;

  // The half-warp walks its hit list (written by the forward pass: the batches it evaluated, each
  // with its tet ids and, per pixel, the bit set of the batch entries the pixel hit) from the last
  // entry to the first.  Batch c holds entries [16 c, 16 c + 16) of the list, the last one fewer.
  const int64_t hbase = (int64_t)u.start * u.subs + (int64_t)u.sub * u.len;
  const int64_t mbase = hbase + 16 * ((int64_t)u.tile * u.subs + u.sub);
  int nmax = (unit < n_units && RM_INDEX_OK((int64_t)u.tile * u.subs + u.sub, RM_X_UNITS, 4))
                 ? min(__ldg(hit_counts + (int64_t)u.tile * u.subs + u.sub), u.len) : 0;
  if (nmax > 0 && !(RM_INDEX_OK(hbase + nmax - 1, RM_X_HIT_IDS, 2) &&
                    RM_INDEX_OK(mbase + (nmax + kChunk - 1) / kChunk * kChunk - 1, RM_X_HIT_MASKS, 3)))
    nmax = 0;
  const int nchunks = (nmax + kChunk - 1) / kChunk;
  const int max_chunks = max(nchunks, __shfl_xor_sync(0xffffffffu, nchunks, 16));

  // chunk k of this half (k = 0 is the LAST batch of its hit list) sits in buffer k&1
  // Tet id and per-pixel bits this lane loads for chunk k+1, fetched while chunk k is issued.
  int id_next = 0;
  unsigned bits_next = 0;
  {
    const int e0 = (nchunks - 1) * kChunk + lane16;
    if (nchunks >= 1) {
      if (e0 < nmax) id_next = __ldg(hit_ids + hbase + e0);
      bits_next = __ldg(hit_masks + mbase + e0);
    }
  }
  auto issue = [&](int k) {
    int c = nchunks - 1 - k;
    unsigned bits = 0u;
    int id = 0;
    if (c >= 0) {
      id = id_next;
      bits = bits_next;
      if (c >= 1) {  // batch c - 1 is a full batch
        const int e = (c - 1) * kChunk + lane16;
        id_next = __ldg(hit_ids + hbase + e);
        bits_next = __ldg(hit_masks + mbase + e);
      }
    }
    // per-pixel bit sets -> per-entry pixel masks (lane j gets the mask of entry j of the batch)
    lane_bits[warp][half][lane16] = bits;
    __syncwarp();
    unsigned m = transpose_masks(lane_bits[warp][half], lane16);
    if (m && !RM_INDEX_OK(id, RM_X_TETS, 1)) m = 0u;  // an id outside the tet table: the entry is dropped
    __syncwarp();
    stage_id[warp][half][k & 1][lane16] = id;
    stage_mask[warp][half][k & 1][lane16] = m;
    if (m) {
      const float4* src = records + kRecStride * (int64_t)id;
      float4* dst = stage[warp][half][k & 1] + lane16 * 6;
#pragma unroll
      for (int q = 0; q < 6; ++q) cp_async16(dst + q, src + q);
    }
    cp_async_commit();
  };
  issue(0);
  for (int k = 0; k < max_chunks; ++k) {
    issue(k + 1);
    cp_async_wait<1>();
    __syncwarp();
    const float4* cur = stage[warp][half][k & 1];
    const int* cur_id = stage_id[warp][half][k & 1];
    const unsigned* cur_mask = stage_mask[warp][half][k & 1];
    // Both halves step in lock-step through their own hit entries, last entry first; a half
    // that runs out idles.  Up to kBwdGroup entries that follow one another and whose pixel
    // masks are disjoint are taken in ONE step: every pixel belongs to at most one of them, so
    // its back-to-front order is untouched, and lanes the first entry would leave idle evaluate
    // the next one.
    unsigned todo = (__ballot_sync(0xffffffffu, cur_mask[lane16] != 0u) >> (16 * half)) & 0xFFFFu;
    while (__any_sync(0xffffffffu, todo != 0u)) {
      int mem[kBwdGroup];            // batch positions of the step's entries
      unsigned mem_mask[kBwdGroup];  // and their pixel masks (0: slot unused)
      unsigned covered = 0u;
      {
        bool open = true;
#pragma unroll
        for (int g = 0; g < kBwdGroup; ++g) {
          mem[g] = 0;
          mem_mask[g] = 0u;
          if (open && todo) {
            const int c = 31 - __clz(todo);
            const unsigned mc = cur_mask[c];
            if (g == 0 || (mc & covered) == 0u) {
              mem[g] = c;
              mem_mask[g] = mc;
              covered |= mc;
              todo &= ~(1u << c);
            } else {
              open = false;
            }
          }
        }
      }
      int j = mem[0];  // the entry this lane evaluates
#pragma unroll
      for (int g = 1; g < kBwdGroup; ++g)
        if ((mem_mask[g] >> lane16) & 1u) j = mem[g];
      const float4* rec = cur + j * 6;
      bool hit = (covered >> lane16) & 1u;
      Eval ev;
      if (hit) {  // same arithmetic as the forward pass, so the test succeeds again
        const float4 pl[4] = {rec[0], rec[1], rec[2], rec[3]};
        hit = slab_test<true>(pl, d, min_t, ev) && integrate(rec, d, min_t, ev);
      }
      const unsigned hits = __ballot_sync(0xffffffffu, hit);
      if (hits == 0) continue;
      // Per lane: gradient of the entering plane (v[0..3] -> row[4*pe..]), of the
      // exit plane (v[4..7] -> row[4*px..]) and of the colour fields (v[8..15] ->
      // row[16..23]); zero for lanes without a hit.
      float v[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) v[q] = 0.0f;
      int pe = -1, px = -1;  // planes that receive v[0..3] / v[4..7]; -1: none
      {
        if (hit) {
          const float4 cbv = rec[5];
          const float dens = cbv.w;
          // undo: state before this tet
          logT += ev.tau;
          const float Tp = __expf(fminf(logT, 46.0517f));
          const float m0 = dens, m1 = dens * (ev.exit + ev.enter) * 0.5f;
          sz -= m0;
          sw -= m1;
          // reverse of the state update
          const float gcr = gr * Tp, gcg = gg * Tp, gcb = gb * Tp;
          const float gT = gr * ev.cr + gg * ev.cg + gb * ev.cb;
          const float g_a = -glogT;
          const float g_m1 = 2.0f * sz * gx + gw;
          const float g_m0 = 2.0f * sw * gy + gz;
          float g_dens = g_m0 + g_m1 * (ev.exit + ev.enter) * 0.5f + gv * 2.0f * dens * ev.dt * (1.0f / 3.0f);
          float g_exit = g_m1 * dens * 0.5f, g_enter = g_exit;
          if (ev.exit - ev.enter > 0.0f) {
            float kk = gv * dens * dens * (1.0f / 3.0f);
            g_exit += kk;
            g_enter -= kk;
          }
          glogT = fmaf(gT, Tp, glogT);
          gz = fmaf(2.0f * m1, gx, gz);
          gw = fmaf(2.0f * m0, gy, gw);
          // reverse of the segment integral
          const float cxr = cbv.x + ev.ox, cxg = cbv.y + ev.ox, cxb = cbv.z + ev.ox;
          const float cer = cbv.x + ev.oe, ceg = cbv.y + ev.oe, ceb = cbv.z + ev.oe;
          const float g_w0 = gcr * cxr + gcg * cxg + gcb * cxb;
          const float g_w1 = gcr * cer + gcg * ceg + gcb * ceb;
          const float G = gcr + gcg + gcb;
          const float wsum = ev.w0 + ev.w1;
          const float g_ox = ev.w0 * G, g_oe = ev.w1 * G;
          const float g_gd = g_ox * (ev.exit + min_t) + g_oe * (ev.enter + min_t);
          g_exit = fmaf(g_ox, ev.gd, g_exit);
          g_enter = fmaf(g_oe, ev.gd, g_enter);
          const float g_phi = g_w0 - g_w1;
          float dphi;  // d phi / d tau = (alpha - phi) / tau = -w0 / tau
          dphi = -__fdividef(ev.w0, ev.tau);
          const float g_tau = g_phi * dphi + g_w0 * ev.alpha + g_a;
          g_dens = fmaf(g_tau, ev.dt, g_dens);
          const float g_dt = g_tau * dens;
          if (ev.exit - ev.enter > 0.0f) {
            g_exit += g_dt;
            g_enter -= g_dt;
          }
          float g_tx = 0.0f, g_te = 0.0f;
          if (ev.tx > ev.enter) g_tx = g_exit; else g_enter += g_exit;
          if (ev.te > 0.0f) g_te = g_enter;
          // planes: t = -D/den - min_t  =>  dt/dD = -1/den, dt/dn = (D/den^2) d
          if (g_te != 0.0f && ev.ie >= 0) {
            const float4 p = rec[ev.ie];
            const float r = __fdividef(1.0f, p.x * d.x + p.y * d.y + p.z * d.z);
            const float kn = g_te * p.w * r * r;
            v[0] = kn * d.x; v[1] = kn * d.y; v[2] = kn * d.z; v[3] = -g_te * r;
            pe = ev.ie;
          }
          if (g_tx != 0.0f && ev.ix >= 0) {
            const float4 p = rec[ev.ix];
            const float r = __fdividef(1.0f, p.x * d.x + p.y * d.y + p.z * d.z);
            const float kn = g_tx * p.w * r * r;
            v[4] = kn * d.x; v[5] = kn * d.y; v[6] = kn * d.z; v[7] = -g_tx * r;
            px = ev.ix;
          }
          v[8] = g_gd * d.x;
          v[9] = g_gd * d.y;
          v[10] = g_gd * d.z;
          v[11] = g_ox + g_oe;
          v[12] = wsum * gcr;
          v[13] = wsum * gcg;
          v[14] = wsum * gcb;
          v[15] = g_dens;
        }
      }
      // Reduction over the pixels of a tile, entry by entry of the step.  If every contributing
      // lane of a half enters through the same face and leaves through the same face, and enough
      // lanes hit, the 16 sums are formed first (shared-memory transpose, one atomic per lane);
      // otherwise each hit lane adds its own 16 values.  `GROUPED` = a half took several entries
      // in this step: the lanes of the other entries then count as lanes without a hit.
      auto reduce_entry = [&](auto grouped, int g) {
        constexpr bool GROUPED = decltype(grouped)::value;
        const bool hit_g = GROUPED ? hit && ((mem_mask[g] >> lane16) & 1u) : hit;
        const unsigned my_hits =
            ((GROUPED ? __ballot_sync(0xffffffffu, hit_g) : hits) >> (16 * half)) & 0xFFFFu;
        const unsigned e_lanes = (__ballot_sync(0xffffffffu, hit_g && pe >= 0) >> (16 * half)) & 0xFFFFu;
        const unsigned x_lanes = (__ballot_sync(0xffffffffu, hit_g && px >= 0) >> (16 * half)) & 0xFFFFu;
        const int src_e = e_lanes ? (__ffs(e_lanes) - 1) + 16 * half : lane;
        const int src_x = x_lanes ? (__ffs(x_lanes) - 1) + 16 * half : lane;
        const int pe_ref = __shfl_sync(0xffffffffu, pe, src_e);
        const int px_ref = __shfl_sync(0xffffffffu, px, src_x);
        const bool odd = hit_g && ((pe >= 0 && pe != pe_ref) || (px >= 0 && px != px_ref));
        const bool sum_over_tile =
            __ballot_sync(0xffffffffu, odd || (my_hits != 0 && __popc(my_hits) < kTileSumMinHits)) == 0;
        if (sum_over_tile) {
          if (GROUPED && __ballot_sync(0xffffffffu, my_hits != 0u) == 0u) return;
          // transpose through shared memory: every lane stores its 16 values as a row (stride 20
          // floats keeps the 128-bit stores aligned and the column reads free of bank conflicts),
          // then lane l adds up column l
          float* rb = reduce_buf[warp] + half * (kChunk * 20 + 16);
          float4* row4 = reinterpret_cast<float4*>(rb + lane16 * 20);
          const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
          row4[0] = (!GROUPED || hit_g) ? make_float4(v[0], v[1], v[2], v[3]) : z4;
          row4[1] = (!GROUPED || hit_g) ? make_float4(v[4], v[5], v[6], v[7]) : z4;
          row4[2] = (!GROUPED || hit_g) ? make_float4(v[8], v[9], v[10], v[11]) : z4;
          row4[3] = (!GROUPED || hit_g) ? make_float4(v[12], v[13], v[14], v[15]) : z4;
          __syncwarp();
          float sum = 0.0f;
#pragma unroll
          for (int r = 0; r < kChunk; ++r) sum += rb[r * 20 + lane16];
          __syncwarp();
          if (my_hits && sum != 0.0f) {
            float* row = grec + (int64_t)cur_id[mem[g]] * 24;
            const int f = lane16;
            const int dst = f < 4 ? 4 * pe_ref + f : (f < 8 ? 4 * px_ref + (f - 4) : f + 8);
            if (dst >= 0) atomicAdd(row + dst, sum);
          }
        } else if (hit_g) {
          // 128-bit reductions: a plane's four sums and the colour sums are 16-byte aligned
          float4* row = reinterpret_cast<float4*>(grec + (int64_t)cur_id[j] * 24);
          if (pe >= 0) atomicAdd(row + pe, make_float4(v[0], v[1], v[2], v[3]));
          if (px >= 0) atomicAdd(row + px, make_float4(v[4], v[5], v[6], v[7]));
          atomicAdd(row + 4, make_float4(v[8], v[9], v[10], v[11]));
          atomicAdd(row + 5, make_float4(v[12], v[13], v[14], v[15]));
        }
      };
      static_assert(kBwdGroup >= 2, "the step takes at least two entries");
      if (!__any_sync(0xffffffffu, mem_mask[1] != 0u)) {
        reduce_entry(std::false_type{}, 0);
      } else {
#pragma unroll
        for (int g = 0; g < kBwdGroup; ++g) {
          if (g > 1 && !__any_sync(0xffffffffu, mem_mask[g] != 0u)) break;
          reduce_entry(std::true_type{}, g);
        }
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
}

// ----------------------------------------------------------------------------
// Densification statistics (slang/alphablend_shader_interp.slang:433-599,
// internal/render_err.py:119-150): the forward walk again, from the pixel centres,
// with the pixel state starting at log-transmittance 1 as the reference has it;
// every hit adds T = exp(logT_before) * optical_depth times (1, err, err^2, ssim,
// entry point, exit point, 1, mid point) to row g of tet_err[T,16] and updates
// tet_count[T,2] (hit count, max of int(65535*T)).  The reference issues 14 float
// and 2 integer atomics per (pixel, tet) hit; here the 16 pixels of a tile are
// summed first (transposed butterfly) when at least four of them hit, else each
// hit pixel issues four 128-bit reductions.
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_tet_err(const int32_t* __restrict__ list, const int2* __restrict__ ranges, const float4* __restrict__ records,
          RmCamera rcam, const float* __restrict__ pixel_err, const float* __restrict__ ssim_err,
          float* __restrict__ tet_err, int32_t* __restrict__ tet_count, int subs, int64_t n_units) {
  __shared__ __align__(16) float4 stage[kWarpsPerBlock][2][2][kChunk * 6];
  __shared__ int stage_id[kWarpsPerBlock][2][2][kChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, lane16 = lane & 15;
  const unsigned half_mask = 0xFFFFu << (16 * half);
  const int64_t unit = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * 2 + half;
  Unit u = make_unit(rcam, ranges, unit, n_units, subs, lane16);

  f3 d = {0.f, 0.f, 1.f};
  const int64_t pix = (int64_t)u.y * rcam.image_width + u.x;
  const float sx = (float)u.x + 0.5f, sy = (float)u.y + 0.5f;
  float perr = 0.f, serr = 0.f;
  if (u.inside) {
    d = ray_direction(rcam, sx, sy);
    perr = __ldg(pixel_err + pix);
    serr = __ldg(ssim_err + pix);
  }
  const float min_t = rcam.min_t;
  const f3 cam = {__ldg(rcam.cam_pos), __ldg(rcam.cam_pos + 1), __ldg(rcam.cam_pos + 2)};
  float X0, X1, Y0, Y1;
  halfwarp_sample_box(u.inside, sx, sy, X0, X1, Y0, Y1);
  const float qnan = __int_as_float(0x7fc00000);
  float4 nq0 = make_float4(qnan, qnan, qnan, qnan), nq1 = nq0, nq2 = nq0;

  float logT = 1.0f, T = 2.718281828f;  // the reference starts the walk at log-transmittance 1
  bool active = u.inside;
  const int nchunks = (u.len + kChunk - 1) / kChunk;
  const int max_chunks = max(nchunks, __shfl_xor_sync(0xffffffffu, nchunks, 16));
  bool fetching = __ballot_sync(0xffffffffu, active) & half_mask;

  if (fetching && lane16 < u.len) {
    int id = __ldg(list + u.start + lane16);
    if (!RM_INDEX_OK(id, RM_X_TETS, 6)) id = 0;
    stage_id[warp][half][0][lane16] = id;
    const float4* src = records + kRecStride * (int64_t)id;
#pragma unroll
    for (int k = 0; k < 6; ++k) cp_async16(stage[warp][half][0] + lane16 * 6 + k, src + k);
    nq0 = __ldg(src + 6);
    nq1 = __ldg(src + 7);
    nq2 = __ldg(src + 8);
  }
  cp_async_commit();
  int id_next = (fetching && kChunk + lane16 < u.len) ? __ldg(list + u.start + kChunk + lane16) : 0;
  if (!RM_INDEX_OK(id_next, RM_X_TETS, 6)) id_next = 0;

  for (int c = 0; c < max_chunks; ++c) {
    float4* cur = stage[warp][half][c & 1];
    float4* nxt = stage[warp][half][(c & 1) ^ 1];
    const int* cur_id = stage_id[warp][half][c & 1];
    const float4 cq0 = nq0, cq1 = nq1, cq2 = nq2;
    {
      int e = (c + 1) * kChunk + lane16;
      if (fetching && e < u.len) {
        stage_id[warp][half][(c & 1) ^ 1][lane16] = id_next;
        const float4* src = records + kRecStride * (int64_t)id_next;
#pragma unroll
        for (int k = 0; k < 6; ++k) cp_async16(nxt + lane16 * 6 + k, src + k);
        nq0 = __ldg(src + 6);
        nq1 = __ldg(src + 7);
        nq2 = __ldg(src + 8);
      }
      cp_async_commit();
      if (fetching && e + kChunk < u.len) id_next = __ldg(list + u.start + e + kChunk);
      if (!RM_INDEX_OK(id_next, RM_X_TETS, 6)) id_next = 0;
    }
    cp_async_wait<1>();
    __syncwarp();
    const bool nonzero = fetching && (c * kChunk + lane16 < u.len) && cur[lane16 * 6 + 5].w > 0.0f &&
                         !hull_misses_box(cq0, cq1, cq2, X0, X1, Y0, Y1);
    unsigned todo = (__ballot_sync(0xffffffffu, nonzero) >> (16 * half)) & 0xFFFFu;
    const int steps = max(__popc(todo), __shfl_xor_sync(0xffffffffu, __popc(todo), 16));
    for (int step = 0; step < steps; ++step) {
      int j = 0;
      bool in_range = false;
      if (todo) {
        j = __ffs(todo) - 1;
        todo &= todo - 1;
        in_range = true;
      }
      const float4* rec = cur + j * 6;
      const float4 pl[4] = {rec[0], rec[1], rec[2], rec[3]};
      bool hit = false;
      Eval ev;
      if (in_range && active) hit = slab_test<false>(pl, d, min_t, ev) && integrate(rec, d, min_t, ev);
      const unsigned hits = __ballot_sync(0xffffffffu, hit);
      if (hits == 0) continue;
      float v[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) v[q] = 0.0f;
      int Ti = 0;
      if (hit) {
        const float Tw = T * ev.tau;
        logT -= ev.tau;
        T *= ev.alpha;
        if (logT < -5.5f) active = false;
        const float a1 = ev.enter + min_t, a2 = ev.exit + min_t, am = 0.5f * (ev.enter + ev.exit) + min_t;
        v[0] = Tw;
        v[1] = Tw * perr;
        v[2] = Tw * perr * perr;
        v[5] = Tw * serr;
        v[6] = Tw * fmaf(a1, d.x, cam.x); v[7] = Tw * fmaf(a1, d.y, cam.y); v[8] = Tw * fmaf(a1, d.z, cam.z);
        v[9] = Tw * fmaf(a2, d.x, cam.x); v[10] = Tw * fmaf(a2, d.y, cam.y); v[11] = Tw * fmaf(a2, d.z, cam.z);
        v[12] = Tw;
        v[13] = Tw * fmaf(am, d.x, cam.x); v[14] = Tw * fmaf(am, d.y, cam.y); v[15] = Tw * fmaf(am, d.z, cam.z);
        Ti = (int)(65535.0f * Tw);
      }
      const unsigned my_hits = (hits >> (16 * half)) & 0xFFFFu;
      int tmax = Ti;
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) tmax = max(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
      const int g = cur_id[j];
      if (my_hits && lane16 == __ffs(my_hits) - 1) {
        atomicAdd(tet_count + 2 * (int64_t)g, __popc(my_hits));
        atomicMax(tet_count + 2 * (int64_t)g + 1, tmax);
      }
      if (max(__popc(hits & 0xFFFFu), __popc(hits >> 16)) >= kTileSumMinHits) {
#pragma unroll
        for (int w = 8; w >= 1; w >>= 1) {
          const bool up = lane16 & w;
#pragma unroll
          for (int i = 0; i < w; ++i) {
            const float send = up ? v[i] : v[i + w];
            const float keep = up ? v[i + w] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, w);
          }
        }
        if (my_hits && v[0] != 0.0f) atomicAdd(tet_err + 16 * (int64_t)g + lane16, v[0]);
      } else if (hit) {
        float4* row = reinterpret_cast<float4*>(tet_err + 16 * (int64_t)g);
        atomicAdd(row + 0, make_float4(v[0], v[1], v[2], 0.0f));
        atomicAdd(row + 1, make_float4(0.0f, v[5], v[6], v[7]));
        atomicAdd(row + 2, make_float4(v[8], v[9], v[10], v[11]));
        atomicAdd(row + 3, make_float4(v[12], v[13], v[14], v[15]));
      }
    }
    __syncwarp();
    unsigned act = __ballot_sync(0xffffffffu, active);
    fetching = act & half_mask;
    if (act == 0) break;
  }
  cp_async_wait<0>();
}

// ----------------------------------------------------------------------------
// Backward of the constant-colour debug renderer, as the reference runs it
// (slang/alphablend_shader.slang:186-277, host side alphablend_tiled_slang.py:131-192): every pixel
// walks its tile list from its last contributor to the first; pairs with alpha < 1/255 are skipped
// (although the forward pass blended them); the state before a tet is recovered by undoing the update
// (transmittance by a division, replaced by 1 when 1 - alpha < 1e-3; distortion state with the weight
// (transmittance after the tet) * alpha); the derivatives of update_alpha_out and evaluate_tetra are taken
// at that recovered state.  A debug path: one lane per pixel, records read straight from global memory,
// gradients added to the record-gradient rows with 128-bit reductions (the reference issues 16 scalar
// atomics per hit); k_backward_finish then applies the chain rule to vertices and (r, g, b, density).
// ----------------------------------------------------------------------------
__device__ __forceinline__ float tukey_power_ladder_dx(float x, float p) {
  if (x == 0.0f) return 0.0f;
  const float q = fmaxf(fabsf(p - 1.0f), 1.0754944e-20f);
  return fabsf(p - 1.0f) / q * __powf(fabsf(x) / q + 1.0f, p - 1.0f);
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_backward_cc(const int32_t* __restrict__ list, const int2* __restrict__ ranges, const float4* __restrict__ records,
              RmCamera rcam, const float4* __restrict__ out_img, const float4* __restrict__ dist_img,
              const int32_t* __restrict__ n_contrib, const float4* __restrict__ g_img,
              const float4* __restrict__ g_dist, float pre_multi, float ladder_p, float* __restrict__ grec, int subs,
              int64_t n_units) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, lane16 = lane & 15;
  const int64_t unit = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * 2 + half;
  Unit u = make_unit(rcam, ranges, unit, n_units, subs, lane16);
  if (!u.inside) return;
  const int64_t pix = (int64_t)u.y * rcam.image_width + u.x;
  const f3 d = ray_direction(rcam, (float)u.x + 0.5f, (float)u.y + 0.5f);
  const float min_t = rcam.min_t;
  float4 st = __ldg(out_img + pix);   // r, g, b, transmittance
  float4 ds = __ldg(dist_img + pix);  // distortion state x, y, z, w
  float4 gi = __ldg(g_img + pix);
  float4 gd = __ldg(g_dist + pix);
  const int last = min(__ldg(n_contrib + pix), u.len);
  for (int j = last - 1; j >= 0; --j) {
    const int id = __ldg(list + u.start + j);
    if (!RM_INDEX_OK(id, RM_X_TETS, 7)) continue;
    const float4* rec = records + kRecStride * (int64_t)id;
    const float4 pl[4] = {__ldg(rec), __ldg(rec + 1), __ldg(rec + 2), __ldg(rec + 3)};
    Eval ev;
    if (!slab_test<true>(pl, d, min_t, ev)) continue;
    const float4 cb = __ldg(rec + 5);  // r, g, b, density
    const float dens = cb.w;
    const float ex = __expf(-dens * ev.dt);
    const float a = fminf(fmaxf(1.0f - ex, 0.0f), 1.0f);
    if (a < 1.0f / 255.0f) continue;
    const float m = tukey_power_ladder(ev.enter * pre_multi, ladder_p);
    // undo
    const float w_u = st.w * a;
    const float Tp = (1.0f - a < 1e-3f) ? 1.0f : st.w / (1.0f - a);
    st.x -= a * cb.x * Tp;
    st.y -= a * cb.y * Tp;
    st.z -= a * cb.z * Tp;
    st.w = Tp;
    ds.z -= w_u;
    ds.w -= w_u * m;
    ds.x -= 2.0f * w_u * m * ds.z;
    ds.y -= 2.0f * w_u * ds.w;
    // reverse of the update at the recovered state
    const float weight = Tp * a;
    const float gcx = gi.x * Tp, gcy = gi.y * Tp, gcz = gi.z * Tp;
    float g_T = a * (gi.x * cb.x + gi.y * cb.y + gi.z * cb.z) + gi.w * (1.0f - a);
    float g_a = -gi.w * Tp;
    const float g_weight = gd.x * 2.0f * m * ds.z + gd.y * 2.0f * ds.w + gd.z + gd.w * m;
    const float g_m = gd.x * 2.0f * weight * ds.z + gd.w * weight;
    gd.z = gd.z + gd.x * 2.0f * weight * m;
    gd.w = gd.w + gd.y * 2.0f * weight;
    g_T += g_weight * a;
    g_a += g_weight * Tp;
    gi.w = g_T;
    float g_enter = g_m * tukey_power_ladder_dx(ev.enter * pre_multi, ladder_p) * pre_multi;
    // reverse of evaluate_tetra
    const float g_alpha = g_a + gcx * cb.x + gcy * cb.y + gcz * cb.z;
    const float inner = 1.0f - ex;
    const float g_tau = (inner > 0.0f && inner < 1.0f) ? g_alpha * ex : 0.0f;
    const float g_dt = g_tau * dens;
    float g_tx = 0.0f;
    if (ev.tx - ev.enter > 0.0f) { g_tx = g_dt; g_enter -= g_dt; }
    const float g_te = ev.te > 0.0f ? g_enter : 0.0f;
    float4* row = reinterpret_cast<float4*>(grec + (int64_t)id * 24);
    if (g_te != 0.0f && ev.ie >= 0) {
      const float4 p = pl[ev.ie];
      const float r = __fdividef(1.0f, p.x * d.x + p.y * d.y + p.z * d.z);
      const float kn = g_te * p.w * r * r;
      atomicAdd(row + ev.ie, make_float4(kn * d.x, kn * d.y, kn * d.z, -g_te * r));
    }
    if (g_tx != 0.0f && ev.ix >= 0) {
      const float4 p = pl[ev.ix];
      const float r = __fdividef(1.0f, p.x * d.x + p.y * d.y + p.z * d.z);
      const float kn = g_tx * p.w * r * r;
      atomicAdd(row + ev.ix, make_float4(kn * d.x, kn * d.y, kn * d.z, -g_tx * r));
    }
    atomicAdd(row + 5, make_float4(gcx * a, gcy * a, gcz * a, g_tau * ev.dt));
  }
}

// Clears the record-gradient rows (6 float4 each) of the tets flagged by the forward pass.
__global__ void __launch_bounds__(256)
k_clear_flagged_rows(const uint8_t* __restrict__ tet_flags, int64_t T, float4* __restrict__ grec) {
  // four tets per thread: one 32-bit load of their flags
  const int64_t g4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (g4 >= T) return;
  uint32_t f4 = 0;
  if (g4 + 4 <= T && (reinterpret_cast<uintptr_t>(tet_flags) & 3) == 0) {
    f4 = *reinterpret_cast<const uint32_t*>(tet_flags + g4);
  } else {
    for (int k = 0; k < 4 && g4 + k < T; ++k) f4 |= (uint32_t)(tet_flags[g4 + k] != 0) << (8 * k);
  }
  if (f4 == 0) return;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if ((f4 >> (8 * k)) & 0xFFu) {
      float4* row = grec + 6 * (g4 + k);
#pragma unroll
      for (int q = 0; q < 6; ++q) row[q] = z;
    }
  }
}

// Chain rule from record gradients to vertices and cell values; one thread per tet.
constexpr int kFinishThreads = 256;

__global__ void __launch_bounds__(kFinishThreads)
k_backward_finish(const int32_t* __restrict__ indices, const float* __restrict__ vertices,
                  const float* __restrict__ cell, int64_t t_begin, int64_t T, RmCamera rcam,
                  const float4* __restrict__ grec, const uint8_t* __restrict__ tet_flags, float* __restrict__ vgrad,
                  float* __restrict__ cgrad) {
  // the block's cell-value gradient rows (7 floats per tet) leave through shared memory as
  // contiguous 16-byte stores
  __shared__ __align__(16) float rows[kFinishThreads * 7];
  const int64_t g0 = t_begin + (int64_t)blockIdx.x * kFinishThreads;  // tets [t_begin, T) are handled by this launch
  const int64_t g = g0 + threadIdx.x;
  float* co = rows + 7 * threadIdx.x;
  float4 q[6];
  bool any = false;
  int4 id = make_int4(0, 0, 0, 0);
  if (g < T && tet_flags[g]) {  // rows of tets without a hit were neither cleared nor written
    // the vertex ids travel with the gradient row: one dependent round trip less before the vertex gathers
    id = __ldg(reinterpret_cast<const int4*>(indices) + g);
#pragma unroll
    for (int k = 0; k < 6; ++k) {
      q[k] = __ldg(grec + 6 * g + k);
      any = any || q[k].x != 0.f || q[k].y != 0.f || q[k].z != 0.f || q[k].w != 0.f;
    }
  }
  if (!any) {
#pragma unroll
    for (int k = 0; k < 7; ++k) co[k] = 0.0f;
  } else {
  f3 cam = {__ldg(rcam.cam_pos), __ldg(rcam.cam_pos + 1), __ldg(rcam.cam_pos + 2)};
  if (!(RM_INDEX_OK(id.x, RM_X_VERTS, 5) && RM_INDEX_OK(id.y, RM_X_VERTS, 5) && RM_INDEX_OK(id.z, RM_X_VERTS, 5) &&
        RM_INDEX_OK(id.w, RM_X_VERTS, 5)))
    id = make_int4(0, 0, 0, 0);
  const int vid[4] = {id.x, id.y, id.z, id.w};
  f3 v[4] = {load3(vertices, id.x), load3(vertices, id.y), load3(vertices, id.z), load3(vertices, id.w)};
  PlaneSetup p;
  make_planes(v, cam, p);
  f3 gvv[4] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int b = i == 3 ? 1 : 0;
    const int e1 = i < 2 ? 1 : 2;
    const int e2 = i == 0 ? 2 : 3;
    const float gD = q[i].w;
    f3 g_n = {q[i].x, q[i].y, q[i].z};
    g_n = g_n + (v[b] - cam) * (-gD);  // D = -n.(b - cam)
    f3 g_b = p.n[i] * (-gD);
    f3 g_raw = g_n * p.sgn[i];
    f3 E1 = v[e1] - v[b], E2 = v[e2] - v[b];
    f3 g_e1 = cross(E2, g_raw);
    f3 g_e2 = cross(g_raw, E1);
    gvv[e1] = gvv[e1] + g_e1;
    gvv[e2] = gvv[e2] + g_e2;
    gvv[b] = gvv[b] + g_b - g_e1 - g_e2;
  }
  const float* c = cell + 7 * g;
  f3 grd = {__ldg(c + 4), __ldg(c + 5), __ldg(c + 6)};
  const float gs0 = q[4].w;
  f3 g_grd = {q[4].x, q[4].y, q[4].z};
  g_grd = g_grd + (cam - v[0]) * gs0;  // s0 = grd.(cam - v0)
  gvv[0] = gvv[0] - grd * gs0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float* vp = vgrad + 3 * (int64_t)vid[k];
    atomicAdd(vp + 0, gvv[k].x);
    atomicAdd(vp + 1, gvv[k].y);
    atomicAdd(vp + 2, gvv[k].z);
  }
  co[0] = __ldg(c) > 0.0f ? q[5].w : 0.0f;
  co[1] = q[5].x;
  co[2] = q[5].y;
  co[3] = q[5].z;
  co[4] = g_grd.x;
  co[5] = g_grd.y;
  co[6] = g_grd.z;
  }
  __syncthreads();
  const int n_rows = (int)min((int64_t)kFinishThreads, T - g0);
  float* dst = cgrad + 7 * g0;  // 7 * 256 floats per block: 16-byte aligned whenever cgrad is
  if (n_rows == kFinishThreads && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    for (int i = threadIdx.x; i < kFinishThreads * 7 / 4; i += kFinishThreads)
      reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(rows)[i];
  } else {
    for (int i = threadIdx.x; i < n_rows * 7; i += kFinishThreads) dst[i] = rows[i];
  }
}

}  // namespace rm

// ----------------------------------------------------------------------------
// host-side launchers used by rm_api.cu
// ----------------------------------------------------------------------------
static inline void unit_grid(const RmCamera* cam, int* subs, int64_t* n_units, unsigned* blocks) {
  int px = cam->tile_width * cam->tile_height;
  *subs = (px + 15) / 16;
  int64_t tiles = (int64_t)(cam->tile_row_end - cam->tile_row_begin) * cam->grid_width;
  *n_units = tiles * *subs;
  int64_t per_block = rm::kWarpsPerBlock * 2;
  *blocks = (unsigned)((*n_units + per_block - 1) / per_block);
}

int rm_launch_pack(const int32_t* indices, const float* vertices, const float* cell, int64_t T, int64_t V,
                   const RmCamera* cam, const int32_t* tiles_touched, float* records, cudaStream_t st) {
  if (T == 0) return RM_OK;
  RmProfScope prof("k_pack_records", st);
  rm_count_launch(), rm::k_pack_records<<<(unsigned)((T + rm::kPackThreads - 1) / rm::kPackThreads), rm::kPackThreads, 0, st>>>(
      indices, vertices, cell, T, V, *cam, tiles_touched, reinterpret_cast<float4*>(records));
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

int rm_launch_forward(const int32_t* list, const int32_t* ranges, const float* records, const RmCamera* cam,
                      const float* jitter, float* out_img, float* dist_img, int32_t* n_contrib, const RmHitList* hits,
                      cudaStream_t st) {
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units == 0) return RM_OK;
  RmProfScope prof("k_forward", st);
  rm_count_launch(), rm::k_forward<false><<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
      list, reinterpret_cast<const int2*>(ranges), reinterpret_cast<const float4*>(records), *cam,
      reinterpret_cast<const float2*>(jitter), reinterpret_cast<float4*>(out_img), dist_img, n_contrib,
      hits ? hits->counts : nullptr, hits ? hits->ids : nullptr, hits ? hits->masks : nullptr,
      hits ? hits->tet_flags : nullptr, subs, n_units, 0.0f, 0.0f);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

int rm_launch_forward_constant_color(const int32_t* list, const int32_t* ranges, const float* records,
                                     const RmCamera* cam, float pre_multi, float ladder_p, float* out_img,
                                     float* dist_img, int32_t* n_contrib, cudaStream_t st) {
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units == 0) return RM_OK;
  RmProfScope prof("k_forward<constant colour>", st);
  rm_count_launch(), rm::k_forward<true><<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
      list, reinterpret_cast<const int2*>(ranges), reinterpret_cast<const float4*>(records), *cam, nullptr,
      reinterpret_cast<float4*>(out_img), dist_img, n_contrib, nullptr, nullptr, nullptr, nullptr, subs, n_units,
      pre_multi, ladder_p);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

int rm_launch_backward_constant_color(const int32_t* list, const int32_t* ranges, const float* records,
                                      const RmCamera* cam, float pre_multi, float ladder_p, const float* out_img,
                                      const float* dist_img, const int32_t* n_contrib, const float* g_img,
                                      const float* g_dist, int64_t T, int64_t V, float* grec, uint8_t* tet_flags,
                                      float* vgrad, cudaStream_t st) {
  RM_CUDA_CHECK(cudaMemsetAsync(vgrad, 0, sizeof(float) * 3 * (size_t)V, st));
  if (T == 0) return RM_OK;
  // every tet may receive a gradient here (the forward pass of this renderer keeps no hit lists)
  RM_CUDA_CHECK(cudaMemsetAsync(grec, 0, sizeof(float) * 24 * (size_t)T, st));
  RM_CUDA_CHECK(cudaMemsetAsync(tet_flags, 1, (size_t)T, st));
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units > 0) {
    RmProfScope prof("k_backward<constant colour>", st);
    rm_count_launch(), rm::k_backward_cc<<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
        list, reinterpret_cast<const int2*>(ranges), reinterpret_cast<const float4*>(records), *cam,
        reinterpret_cast<const float4*>(out_img), reinterpret_cast<const float4*>(dist_img), n_contrib,
        reinterpret_cast<const float4*>(g_img), reinterpret_cast<const float4*>(g_dist), pre_multi, ladder_p, grec, subs,
        n_units);
  }
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

int rm_launch_tet_err(const int32_t* list, const int32_t* ranges, const float* records, const RmCamera* cam,
                      const float* pixel_err, const float* ssim_err, int64_t T, float* tet_err, int32_t* tet_count,
                      cudaStream_t st) {
  if (T == 0) return RM_OK;
  RM_CUDA_CHECK(cudaMemsetAsync(tet_err, 0, sizeof(float) * 16 * (size_t)T, st));
  RM_CUDA_CHECK(cudaMemsetAsync(tet_count, 0, sizeof(int32_t) * 2 * (size_t)T, st));
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units == 0) return RM_OK;
  RmProfScope prof("k_tet_err", st);
  rm_count_launch(), rm::k_tet_err<<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
      list, reinterpret_cast<const int2*>(ranges), reinterpret_cast<const float4*>(records), *cam, pixel_err,
      ssim_err, tet_err, tet_count, subs, n_units);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// Everything of the backward pass except the per-tet chain rule: clears vertices_grad and the
// record-gradient rows of flagged tets, then accumulates the record gradients.
int rm_launch_backward_integrate(const int32_t* ranges, const float* records, const RmCamera* cam, const float* jitter,
                                 const float* out_img, const float* dist_img, const RmHitList* hits, const float* g_img,
                                 const float* g_dist, int64_t T, int64_t V, float* grec, float* vgrad,
                                 cudaStream_t st) {
  RM_CUDA_CHECK(cudaMemsetAsync(vgrad, 0, sizeof(float) * 3 * (size_t)V, st));
  if (T == 0) return RM_OK;
  {
    RmProfScope prof("k_clear_flagged_rows", st);
    rm_count_launch(), rm::k_clear_flagged_rows<<<(unsigned)(((T + 3) / 4 + 255) / 256), 256, 0, st>>>(
        hits->tet_flags, T, reinterpret_cast<float4*>(grec));
  }
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units > 0) {
    RmProfScope prof("k_backward", st);
    rm_count_launch(), rm::k_backward<<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
        reinterpret_cast<const int2*>(ranges), reinterpret_cast<const float4*>(records), *cam,
        reinterpret_cast<const float2*>(jitter), reinterpret_cast<const float4*>(out_img), dist_img, hits->counts,
        hits->ids, hits->masks, reinterpret_cast<const float4*>(g_img), g_dist, grec, subs, n_units);
  }
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// The chain rule from record gradients to vertices and cell values for tets [t_begin, t_end).
int rm_launch_backward_finish(const int32_t* indices, const float* vertices, const float* cell, int64_t t_begin,
                              int64_t t_end, const RmCamera* cam, const float* grec, const RmHitList* hits,
                              float* vgrad, float* cgrad, cudaStream_t st) {
  if (t_end <= t_begin) return RM_OK;
  RmProfScope prof("k_backward_finish", st);
  rm_count_launch(), rm::k_backward_finish<<<(unsigned)((t_end - t_begin + rm::kFinishThreads - 1) / rm::kFinishThreads),
                                            rm::kFinishThreads, 0, st>>>(
      indices, vertices, cell, t_begin, t_end, *cam, reinterpret_cast<const float4*>(grec), hits->tet_flags, vgrad,
      cgrad);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// ----------------------------------------------------------------------------
// rm_backward_static_scratch: the backward pass for callers that may not
// allocate device memory.  Its only scratch, the per-tet record-gradient rows,
// lives in the file-scope device array below instead of a caller buffer.
// ----------------------------------------------------------------------------
#include <mutex>

static __device__ __align__(256) float g_static_grad_records[(size_t)RM_STATIC_SCRATCH_MAX_TETS * RM_GRAD_RECORD_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_addr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int rm_backward_static_scratch(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges,
                                          const float* records, const RmCamera* cam, const float* ray_jitter,
                                          const float* output_img, const float* distortion_img,
                                          const int32_t* n_contributors, const RmHitList* hits,
                                          const float* grad_output_img,
                                          const float* grad_distortion_img, const int32_t* indices,
                                          const float* vertices, const float* cell_values, int64_t n_tets,
                                          int64_t n_vertices, float* vertices_grad, float* cell_values_grad,
                                          void* stream) {
  // the same host-side checks as rm_backward, before anything touches the device
  rm_clear_last_error();
  if (n_tets > RM_STATIC_SCRATCH_MAX_TETS) return RM_ERR_STATIC_SCRATCH;
  int rc = rm_check_cam(cam);
  if (rc) return rc;
  if (n_tets < 0 || n_vertices < 0) return RM_ERR_INVALID_ARG;
  if (!tile_ranges || !ray_jitter || !output_img || !distortion_img || !hits || !hits->counts || !hits->ids ||
      !hits->masks || !hits->tet_flags || !grad_output_img || !grad_distortion_img || !vertices_grad)
    return RM_ERR_INVALID_ARG;
  (void)sorted_tetra_idx;
  (void)n_contributors;
  if (n_tets > 0 && (!indices || !vertices || !cell_values || !cell_values_grad || !records))
    return RM_ERR_INVALID_ARG;
  if (!rm_aligned16(output_img) || !rm_aligned16(grad_output_img) || !rm_aligned16(records) || !rm_aligned16(indices))
    return RM_ERR_WORKSPACE;
  rc = rm_bind_device(vertices_grad);  // makes the device that owns the buffers current
  if (rc) return rc;
  // Set-up, once per device, with that device current: the array's name is a
  // host-side handle, the kernels need its device address.
  int dev = -1;
  RM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return RM_ERR_INVALID_ARG;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) {
      void* addr = nullptr;
      RM_CUDA_CHECK(cudaGetSymbolAddress(&addr, g_static_grad_records));
      g_static_addr[dev] = static_cast<float*>(addr);
    }
    scratch = g_static_addr[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps the previous call's sums: clear the rows this call accumulates into.
  RM_CUDA_CHECK(cudaMemsetAsync(vertices_grad, 0, sizeof(float) * 3 * (size_t)n_vertices, st));
  if (n_tets == 0) return RM_OK;
  {
    RmProfScope prof("k_clear_flagged_rows", st);
    rm_count_launch(), rm::k_clear_flagged_rows<<<(unsigned)(((n_tets + 3) / 4 + 255) / 256), 256, 0, st>>>(
        hits->tet_flags, n_tets, reinterpret_cast<float4*>(scratch));
  }
  int subs;
  int64_t n_units;
  unsigned blocks;
  unit_grid(cam, &subs, &n_units, &blocks);
  if (n_units > 0) {
    RmProfScope prof("k_backward", st);
    rm_count_launch(), rm::k_backward<<<blocks, rm::kWarpsPerBlock * 32, 0, st>>>(
        reinterpret_cast<const int2*>(tile_ranges), reinterpret_cast<const float4*>(records), *cam,
        reinterpret_cast<const float2*>(ray_jitter), reinterpret_cast<const float4*>(output_img), distortion_img,
        hits->counts, hits->ids, hits->masks, reinterpret_cast<const float4*>(grad_output_img), grad_distortion_img,
        scratch, subs, n_units);
  }
  RmProfScope prof2("k_backward_finish", st);
  rm_count_launch(), rm::k_backward_finish<<<(unsigned)((n_tets + rm::kFinishThreads - 1) / rm::kFinishThreads), rm::kFinishThreads, 0, st>>>(
      indices, vertices, cell_values, 0, n_tets, *cam, reinterpret_cast<const float4*>(scratch), hits->tet_flags,
      vertices_grad, cell_values_grad);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// Bounds-checked build: extents of the caller-owned arrays of the integration stages (the entry points
// of these stages carry no array lengths) and the status word of this translation unit.
unsigned rm_bounds_status_raster() { return rm_take_bounds_status(); }
void rm_debug_extent_raster(int which, long long n) {
  if (which >= 0 && which < RM_X_COUNT) rm_set_extent(which, n, nullptr);
#ifdef RM_BOUNDS_CHECK
  cudaDeviceSynchronize();
#endif
}
