// Stage 1 on the GPU: per-tet projection, near-plane clipping, planar/behind
// culling, fp64 circumsphere power (the sort depth), tile rectangle and tile
// count; plus its reverse pass with respect to the vertices.
//
// This translation unit is compiled with -fmad=false: the tile rectangles and
// the sort depth decide the tile lists, which must be bit-identical to the CPU
// restatement of the reference arithmetic, so every fp32/fp64 operation here is
// the plain IEEE operation in the order written.
//
// Reference behaviour reproduced: slang/vertex_shader.slang:20-89,
// slang/camera.slang:103-108,351-508, slang/intersect.slang:76-89,
// slang/stable_power.slang:17-84, slang/utils.slang:85-125.

#include "rm_common.cuh"

namespace rm {

__device__ __forceinline__ float safe_clipf(float v, float lo, float hi) { return fmaxf(fminf(v, hi), lo); }
__device__ __forceinline__ float safe_divf(float a, float b) {
  const float TINY = 1.0754944e-20f;
  if (fabsf(b) < TINY) return safe_clipf(a / TINY, -1e20f, 1e20f);
  return safe_clipf(a / b, -1e20f, 1e20f);
}
__device__ __forceinline__ f3 normalize3(f3 a) {
  float l = sqrtf(dot(a, a));
  return {a.x / l, a.y / l, a.z / l};
}
__device__ __forceinline__ f3 lerp3(f3 a, f3 b, float t) { return a + (b - a) * t; }

__device__ __forceinline__ float dist_norm2(const DevCam& c) {
  return c.dist[0] * c.dist[0] + c.dist[1] * c.dist[1] + c.dist[2] * c.dist[2] + c.dist[3] * c.dist[3];
}

__device__ __forceinline__ f3 point2camspace(f3 p, const DevCam& c) {
  float h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    h[i] = c.W[4 * i + 0] * p.x + c.W[4 * i + 1] * p.y + c.W[4 * i + 2] * p.z + c.W[4 * i + 3] * 1.0f;
  // A rigid world-to-camera transform has the last row (0, 0, 0, 1): w is exactly 1 and x / 1 is x, so
  // the three guarded divisions reduce to the clip (same bits, far fewer instructions).
  if (h[3] == 1.0f) return {safe_clipf(h[0], -1e20f, 1e20f), safe_clipf(h[1], -1e20f, 1e20f), safe_clipf(h[2], -1e20f, 1e20f)};
  return {safe_divf(h[0], h[3]), safe_divf(h[1], h[3]), safe_divf(h[2], h[3])};
}

__device__ __forceinline__ void distort(float& x, float& y, const DevCam& c) {
  if (dist_norm2(c) < 1e-9f) return;
  float k1 = c.dist[0], k2 = c.dist[1], p1 = c.dist[2], p2 = c.dist[3];
  float r2 = x * x + y * y;
  float radial = r2 * (k1 + r2 * k2);
  float tx = 2.0f * p1 * x * y + p2 * (r2 + 2.0f * x * x);
  float ty = 2.0f * p2 * x * y + p1 * (r2 + 2.0f * y * y);
  float nx = x + x * radial + tx;
  float ny = y + y * radial + ty;
  x = nx;
  y = ny;
}

// Fisheye angle functions with a fixed operation sequence (IEEE double, no contraction), so
// that tile rectangles of fisheye cameras are reproducible bit for bit by any implementation
// that evaluates the same series; the result is rounded to float once.  Library acosf/sinf
// differ between vendors in the last bit.
//   asin(s) = sum_n c_n s^(2n+1), c_0 = 1, c_{n+1} = c_n (2n+1)^2 / ((2n+2)(2n+3)), |s| <= 0.5
//   acos(x) = pi/2 - asin(x) for x < 0.5, 2 asin(sqrt((1 - x)/2)) otherwise        (0 <= x <= 1)
//   sin(t)  = sum_n (-1)^n t^(2n+1)/(2n+1)!,                                        0 <= t <= pi/2
__device__ __forceinline__ double asin_series(double s) {
  const double s2 = s * s;
  double term = s, sum = s;
  for (int n = 0; n < 20; ++n) {
    const double a = double(2 * n + 1);
    term = term * s2 * (a * a / (double(2 * n + 2) * double(2 * n + 3)));
    sum += term;
  }
  return sum;
}
__device__ __forceinline__ float fisheye_acos(float x) {
  const double xd = double(x);
  if (xd < 0.5) return float(1.5707963267948966 - asin_series(xd));
  return float(2.0 * asin_series(sqrt((1.0 - xd) * 0.5)));
}
__device__ __forceinline__ float fisheye_sin(float t) {
  const double td = double(t), t2 = td * td;
  double term = td, sum = td;
  for (int n = 1; n < 13; ++n) {
    term = -(term * t2) / (double(2 * n) * double(2 * n + 1));
    sum += term;
  }
  return float(sum);
}

__device__ __forceinline__ f3 camspace_to_image(f3 p, const DevCam& c) {
  float ux, uy;
  if (c.type == 1) {
    f3 dir = normalize3(p);
    float sat = fminf(fmaxf(dir.z, 0.0f), 1.0f);
    float theta = fisheye_acos(sat);
    float st = fisheye_sin(theta);
    float k = (st < 1e-6f) ? 1.0f : theta / st;
    ux = dir.x * k;
    uy = dir.y * k;
  } else {
    ux = p.x / p.z;
    uy = p.y / p.z;
  }
  distort(ux, uy, c);
  float px = ux * c.K[0] + c.K[2];
  float py = uy * c.K[4] + c.K[5];
  return {px, py, p.z};
}

__device__ __forceinline__ void update_bounds_from_edge(f3 a, f3 b, f3& mn, f3& mx, const DevCam& c) {
  int n = 2;
  bool distorted = dist_norm2(c) > 1e-9f;
  if (c.type == 1) n = 4;
  else if (distorted) n = 3;
  for (int i = 0; i < n; ++i) {
    float t = float(i) / float(n - 1);
    f3 s = lerp3(a, b, t);
    f3 pv = camspace_to_image(s, c);
    mn = {fminf(mn.x, pv.x), fminf(mn.y, pv.y), fminf(mn.z, pv.z)};
    mx = {fmaxf(mx.x, pv.x), fmaxf(mx.y, pv.y), fmaxf(mx.z, pv.z)};
  }
}

__device__ __forceinline__ void find_extent(const f3 tet[4], f3& mn, f3& mx, const DevCam& c) {
  const float BIG = 1e20f;
  mn = {BIG, BIG, BIG};
  mx = {-BIG, -BIG, -BIG};
  const float eps = 1e-4f;
#pragma unroll
  for (int f = 0; f < 4; ++f) {
    // faces (0,1,2) (0,2,3) (0,3,1) (1,3,2)
    f3 fv[3];
    if (f == 0) { fv[0] = tet[0]; fv[1] = tet[1]; fv[2] = tet[2]; }
    else if (f == 1) { fv[0] = tet[0]; fv[1] = tet[2]; fv[2] = tet[3]; }
    else if (f == 2) { fv[0] = tet[0]; fv[1] = tet[3]; fv[2] = tet[1]; }
    else { fv[0] = tet[1]; fv[1] = tet[3]; fv[2] = tet[2]; }
    f3 out[4];
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      f3 va = fv[j], vb = fv[(j + 1) % 3];
      bool ain = va.z > eps, bin = vb.z > eps;
      if (ain) {
        bool found = false;
        for (int k = 0; k < cnt; ++k)
          if (out[k].x == va.x && out[k].y == va.y && out[k].z == va.z) found = true;
        if (!found) out[cnt++] = va;
      }
      if (ain != bin) {
        float t = (eps - va.z) / (vb.z - va.z);
        out[cnt++] = lerp3(va, vb, t);
      }
    }
    if (cnt > 1)
      for (int j = 0; j < cnt; ++j) update_bounds_from_edge(out[j], out[(j + 1) % cnt], mn, mx, c);
  }
}

// Extent of a tet that lies entirely in front of the near plane, seen by an
// undistorted pinhole camera.  The general routine then clips nothing and samples
// every directed face edge a->b at its two ends, a + (b-a)*0 and a + (b-a)*1.  The
// first is the vertex a itself (up to the sign of a zero, which no later step can
// see).  The second equals b bit for bit unless the subtraction or the addition
// rounded, which happens for about one sample in forty; its projection is then
// already among the four vertex projections.  So the four vertices are projected,
// the twelve end samples are formed and compared with their vertex, and only the
// ones that differ are projected as well: the same minima and maxima as the 24
// projections of the general routine.
__device__ __forceinline__ void find_extent_unclipped(const f3 cs[4], f3& mn, f3& mx, const DevCam& c) {
  const float BIG = 1e20f;
  mn = {BIG, BIG, BIG};
  mx = {-BIG, -BIG, -BIG};
  auto add = [&](f3 p) {
    const float ux = p.x / p.z, uy = p.y / p.z;
    const float px = ux * c.K[0] + c.K[2];
    const float py = uy * c.K[4] + c.K[5];
    mn = {fminf(mn.x, px), fminf(mn.y, py), fminf(mn.z, p.z)};
    mx = {fmaxf(mx.x, px), fmaxf(mx.y, py), fmaxf(mx.z, p.z)};
  };
  add(cs[0]);
  add(cs[1]);
  add(cs[2]);
  add(cs[3]);
  // directed edges of the faces (0,1,2) (0,2,3) (0,3,1) (1,3,2), two bits per end point
  constexpr unsigned kFrom = 0u | (1u << 2) | (2u << 4) | (0u << 6) | (2u << 8) | (3u << 10) | (0u << 12) | (3u << 14) |
                             (1u << 16) | (1u << 18) | (3u << 20) | (2u << 22);
  constexpr unsigned kTo = 1u | (2u << 2) | (0u << 4) | (2u << 6) | (3u << 8) | (0u << 10) | (3u << 12) | (1u << 14) |
                           (0u << 16) | (3u << 18) | (2u << 20) | (1u << 22);
  unsigned pending = 0;
#pragma unroll
  for (int e = 0; e < 12; ++e) {
    const f3 a = cs[(kFrom >> (2 * e)) & 3u], b = cs[(kTo >> (2 * e)) & 3u];
    const f3 s_ = lerp3(a, b, 1.0f);
    if (s_.x != b.x || s_.y != b.y || s_.z != b.z) pending |= 1u << e;
  }
  while (pending) {
    const int e = __ffs(pending) - 1;
    pending &= pending - 1;
    const unsigned ia = (kFrom >> (2 * e)) & 3u, ib = (kTo >> (2 * e)) & 3u;
    const f3 a = ia == 0 ? cs[0] : (ia == 1 ? cs[1] : (ia == 2 ? cs[2] : cs[3]));
    const f3 b = ib == 0 ? cs[0] : (ib == 1 ? cs[1] : (ib == 2 ? cs[2] : cs[3]));
    add(lerp3(a, b, 1.0f));
  }
}

__device__ __forceinline__ bool is_planar(const f3 v[4]) {
  f3 n = normalize3(cross(v[1] - v[0], v[2] - v[0]));
  float d = dot(n, v[3] - v[0]);
  return fabsf(d) < 1e-3f;
}

__device__ __forceinline__ double length3(d3 a) { return sqrt(dot(a, a)); }

// branch: 0 regular, 1 tiny tet (centroid rule), 2 degenerate (-1e20)
__device__ __forceinline__ double power_of_circumsphere(d3 A, d3 B, d3 C, d3 D, d3 P, d3& center, int& branch) {
  d3 a = B - A, b = C - A, c = D - A;
  double aa = dot(a, a), bb = dot(b, b), cc = dot(c, c);
  d3 cbc = cross(b, c), cca = cross(c, a), cab = cross(a, b);
  double denominator = 2.0 * dot(a, cbc);
  double radius;
  if (fabs(denominator) < 1e-10) {
    double m = fmax(length3(B - A),
                    fmax(length3(C - A), fmax(length3(D - A), fmax(length3(C - B), fmax(length3(D - B), length3(D - C))))));
    if (m < 1e-7) {
      center = (A + B + C + D) * 0.25;
      double dA = length3(A - center), dB = length3(B - center), dC = length3(C - center), dD = length3(D - center);
      radius = fmin(dA, fmin(dB, fmin(dC, dD)));
      d3 diff = center - P;
      branch = 1;
      return dot(diff, diff) - radius * radius;
    }
    branch = 2;
    return -1e20;
  }
  d3 num = cbc * aa + cca * bb + cab * cc;
  d3 rel = {num.x / denominator, num.y / denominator, num.z / denominator};
  center = A + rel;
  radius = length3(rel);
  d3 diff = center - P;
  branch = 0;
  return dot(diff, diff) - radius * radius;
}

__device__ __forceinline__ float clipf(float v, float lo, float hi) { return fmaxf(lo, fminf(hi, v)); }

// One thread per tet (and, for the NaN scan, per vertex coordinate).
// Besides the reference outputs it feeds the binning stages:
//   depth_keys[g]  sortable depth bits, 0xFFFFFFFF for culled tets
//   order_in[g]    g
//   tile_diff      2-D difference array of tile coverage ((gh+1) x (gw+1) int32)
__global__ void __launch_bounds__(256, 4)
k_project(const int32_t* __restrict__ indices, int64_t T, const float* __restrict__ vertices, int64_t V,
          RmCamera rcam, int32_t* __restrict__ tiles_touched, int4* __restrict__ rect, float* __restrict__ vs_tetra,
          float* __restrict__ circumcenter, uint32_t* __restrict__ depth_keys, uint32_t* __restrict__ order_in,
          int32_t* __restrict__ tile_diff, RmBinInfo* __restrict__ info) {
  int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g < 3 * V) {
    float v = __ldg(vertices + g);
    if (v != v) atomicOr(&info->status, RM_STATUS_NAN_VERTEX);
  }
  if (g >= T) return;
  DevCam cam;
  load_cam(rcam, cam);

  int n_tiles = 0;
  int4 r = make_int4(0, 0, 0, 0);
  float depth = 0.0f;
  float ccx = 0.0f, ccy = 0.0f, ccz = 0.0f;

  int4 id = __ldg(reinterpret_cast<const int4*>(indices) + g);
  // A vertex id outside [0, V) would read out of bounds here and in every later stage: the tet is
  // culled (later stages skip culled tets) and the host is told through the status word.
  const bool ids_ok = (uint32_t)id.x < (uint64_t)V && (uint32_t)id.y < (uint64_t)V && (uint32_t)id.z < (uint64_t)V &&
                      (uint32_t)id.w < (uint64_t)V;
  if (!ids_ok) {
    atomicOr(&info->status, RM_STATUS_BAD_INDEX);
    id = make_int4(0, 0, 0, 0);
  }
  f3 v[4] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}};
  if (ids_ok) {
    v[0] = load3(vertices, id.x);
    v[1] = load3(vertices, id.y);
    v[2] = load3(vertices, id.z);
    v[3] = load3(vertices, id.w);
  }
  do {
    if (!ids_ok) break;
    if (is_planar(v)) break;
    f3 cs[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) cs[k] = point2camspace(v[k], cam);
    f3 mn, mx;
    const bool simple = cam.type == 0 && dist_norm2(cam) < 1e-9f && cs[0].z > 1e-4f && cs[1].z > 1e-4f &&
                        cs[2].z > 1e-4f && cs[3].z > 1e-4f;
    if (simple && (cam.row0 > 0 || cam.row1 < cam.grid_h)) {
      // Band pre-test: a tet whose four projected vertices all lie more than a pixel above the band's
      // first pixel row, or more than a pixel below its last, ends with an empty rectangle after the
      // clamp below; it is culled here, before the extent and the fp64 circumsphere.  The comparison
      // py < y is made without the division (Z > 0): fy*Y + (cy - y)*Z < 0; its rounding error is far
      // below the one-pixel margin wherever py is near y.
      const float c_lo = cam.K[5] - (float(cam.row0 * cam.tile_h) - 1.0f);
      const float c_hi = cam.K[5] - (float(cam.row1 * cam.tile_h) + 1.0f);
      bool above = true, below = true;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = cam.K[4] * cs[k].y;
        above = above && (a + c_lo * cs[k].z < 0.0f);
        below = below && (a + c_hi * cs[k].z > 0.0f);
      }
      if (above || below) break;
    }
    if (simple) find_extent_unclipped(cs, mn, mx, cam);
    else find_extent(cs, mn, mx, cam);
    if (mx.z <= 0.0f) break;
    d3 A = {v[0].x, v[0].y, v[0].z}, B = {v[1].x, v[1].y, v[1].z}, C = {v[2].x, v[2].y, v[2].z},
       D = {v[3].x, v[3].y, v[3].z}, P = {cam.pos[0], cam.pos[1], cam.pos[2]};
    d3 cc = {0, 0, 0};
    int branch;
    float sort_depth = float(power_of_circumsphere(A, B, C, D, P, cc, branch));
    if (sort_depth < -1e19f) break;
    int min_x = int(floorf(clipf(mn.x / float(cam.tile_w), 0.f, float(cam.grid_w))));
    int min_y = int(floorf(clipf(mn.y / float(cam.tile_h), 0.f, float(cam.grid_h))));
    int max_x = int(ceilf(clipf(mx.x / float(cam.tile_w), 0.f, float(cam.grid_w))));
    int max_y = int(ceilf(clipf(mx.y / float(cam.tile_h), 0.f, float(cam.grid_h))));
    // band restriction (whole frame: row0 = 0, row1 = grid_h)
    min_y = max(min_y, cam.row0);
    max_y = min(max_y, cam.row1);
    if (max_y < min_y) max_y = min_y;
    int nt = (max_x - min_x) * (max_y - min_y);
    if (nt == 0) break;
    n_tiles = nt;
    r = make_int4(min_x, min_y, max_x, max_y);
    depth = fminf(fmaxf(sort_depth, -1e20f), 1e20f);
    ccx = float(cc.x);
    ccy = float(cc.y);
    ccz = float(cc.z);
  } while (false);

  tiles_touched[g] = n_tiles;
  rect[g] = r;
  vs_tetra[3 * g + 0] = 0.0f;
  vs_tetra[3 * g + 1] = 0.0f;
  vs_tetra[3 * g + 2] = depth;
  circumcenter[3 * g + 0] = ccx;
  circumcenter[3 * g + 1] = ccy;
  circumcenter[3 * g + 2] = ccz;
  depth_keys[g] = n_tiles > 0 ? float2sortable_key(depth) : 0xFFFFFFFFu;
  order_in[g] = (uint32_t)g;
  if (n_tiles > 0) {
    const int pitch = cam.grid_w + 1;
    atomicAdd(&tile_diff[r.y * pitch + r.x], 1);
    atomicAdd(&tile_diff[r.y * pitch + r.z], -1);
    atomicAdd(&tile_diff[r.w * pitch + r.x], -1);
    atomicAdd(&tile_diff[r.w * pitch + r.z], 1);
  }
  // visible-tet count, one atomic per warp
  unsigned m = __ballot_sync(__activemask(), n_tiles > 0);
  if (m && (threadIdx.x & 31) == (__ffs(m) - 1)) atomicAdd(&info->n_visible, __popc(m));
}

// Reverse of the sort-depth / circumcentre computation with respect to the
// four vertices, in fp64, accumulated into vertices_grad with fp32 atomics.
__global__ void __launch_bounds__(256)
k_vertex_backward(const int32_t* __restrict__ indices, const float* __restrict__ vertices, int64_t T, RmCamera rcam,
                  const int32_t* __restrict__ tiles_touched, const float* __restrict__ g_vs,
                  const float* __restrict__ g_cc, float* __restrict__ vgrad) {
  int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= T) return;
  if (tiles_touched[g] == 0) return;
  float gp_in = __ldg(g_vs + 3 * g + 2);
  float gc0 = __ldg(g_cc + 3 * g), gc1 = __ldg(g_cc + 3 * g + 1), gc2 = __ldg(g_cc + 3 * g + 2);
  if (gp_in == 0.0f && gc0 == 0.0f && gc1 == 0.0f && gc2 == 0.0f) return;
  int4 id = __ldg(reinterpret_cast<const int4*>(indices) + g);
  int vid[4] = {id.x, id.y, id.z, id.w};
  d3 p[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f3 v = load3(vertices, vid[k]);
    p[k] = {v.x, v.y, v.z};
  }
  d3 P = {__ldg(rcam.cam_pos), __ldg(rcam.cam_pos + 1), __ldg(rcam.cam_pos + 2)};
  d3 center = {0, 0, 0};
  int branch;
  double power = power_of_circumsphere(p[0], p[1], p[2], p[3], P, center, branch);
  float sd = float(power);
  double g_power = (sd > -1e20f && sd < 1e20f) ? double(gp_in) : 0.0;
  d3 g_center = {gc0, gc1, gc2};
  d3 gp[4] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
  if (branch == 0) {
    d3 a = p[1] - p[0], b = p[2] - p[0], c = p[3] - p[0];
    double aa = dot(a, a), bb = dot(b, b), cc = dot(c, c);
    d3 X = cross(b, c), Y = cross(c, a), Z = cross(a, b);
    double den = 2.0 * dot(a, X);
    d3 num = X * aa + Y * bb + Z * cc;
    d3 rel = {num.x / den, num.y / den, num.z / den};
    d3 diff = center - P;
    d3 g_ct = g_center + diff * (2.0 * g_power);
    d3 g_rel = g_ct - rel * (2.0 * g_power);
    d3 g_num = {g_rel.x / den, g_rel.y / den, g_rel.z / den};
    double g_den = -dot(g_rel, rel) / den;
    double g_aa = dot(g_num, X), g_bb = dot(g_num, Y), g_cc2 = dot(g_num, Z);
    d3 g_X = g_num * aa + a * (2.0 * g_den);
    d3 g_Y = g_num * bb, g_Z = g_num * cc;
    d3 g_a = X * (2.0 * g_den) + a * (2.0 * g_aa);
    d3 g_b = b * (2.0 * g_bb);
    d3 g_c = c * (2.0 * g_cc2);
    g_b = g_b + cross(c, g_X);  g_c = g_c + cross(g_X, b);
    g_c = g_c + cross(a, g_Y);  g_a = g_a + cross(g_Y, c);
    g_a = g_a + cross(b, g_Z);  g_b = g_b + cross(g_Z, a);
    gp[1] = g_a; gp[2] = g_b; gp[3] = g_c;
    gp[0] = g_ct - g_a - g_b - g_c;
  } else if (branch == 1) {
    d3 diff = center - P;
    d3 g_ct = g_center + diff * (2.0 * g_power);
    int arg = 0;
    double best = length3(p[0] - center);
#pragma unroll
    for (int k = 1; k < 4; ++k) {
      double dk = length3(p[k] - center);
      if (dk < best) { best = dk; arg = k; }
    }
    d3 g_rv = (p[arg] - center) * (-2.0 * g_power);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k == arg) gp[k] = gp[k] + g_rv;
    }
    g_ct = g_ct - g_rv;
#pragma unroll
    for (int k = 0; k < 4; ++k) gp[k] = gp[k] + g_ct * 0.25;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    atomicAdd(vgrad + 3 * (int64_t)vid[k] + 0, float(gp[k].x));
    atomicAdd(vgrad + 3 * (int64_t)vid[k] + 1, float(gp[k].y));
    atomicAdd(vgrad + 3 * (int64_t)vid[k] + 2, float(gp[k].z));
  }
}

}  // namespace rm

// ---------------------------------------------------------------------------
// host-side launchers used by rm_api.cu
// ---------------------------------------------------------------------------
int rm_launch_project(const int32_t* indices, int64_t T, const float* vertices, int64_t V, const RmCamera* cam,
                      int32_t* tiles_touched, int32_t* rect, float* vs_tetra, float* circumcenter,
                      uint32_t* depth_keys, uint32_t* order_in, int32_t* tile_diff, RmBinInfo* info,
                      cudaStream_t st) {
  int64_t n = T > 3 * V ? T : 3 * V;
  if (n == 0) return RM_OK;
  unsigned blocks = (unsigned)((n + 255) / 256);
  RmProfScope prof("k_project", st);
  rm_count_launch(), rm::k_project<<<blocks, 256, 0, st>>>(indices, T, vertices, V, *cam, tiles_touched, reinterpret_cast<int4*>(rect),
                                        vs_tetra, circumcenter, depth_keys, order_in, tile_diff, info);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

int rm_launch_vertex_backward(const int32_t* indices, const float* vertices, int64_t T, const RmCamera* cam,
                              const int32_t* tiles_touched, const float* g_vs, const float* g_cc, float* vgrad,
                              cudaStream_t st) {
  if (T == 0) return RM_OK;
  unsigned blocks = (unsigned)((T + 255) / 256);
  RmProfScope prof("k_vertex_backward", st);
  rm_count_launch(), rm::k_vertex_backward<<<blocks, 256, 0, st>>>(indices, vertices, T, *cam, tiles_touched, g_vs, g_cc, vgrad);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}
