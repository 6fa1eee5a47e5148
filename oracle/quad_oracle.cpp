// CPU restatement of the reference's brute-force quadrature renderer
// (jaxutil/tetra_quad.py), the reference's own CPU path for a tetrahedral
// field: density at a point = sum of the densities of the tets containing it,
// colour = density-weighted mean of base + grd.(x - v0).
//
// TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); never part of the
// product path.  PARITY UNPINNED: JAX is not installed where this was written,
// so the restatement could not be run against the original.
//
// One deliberate deviation, selectable at run time: the reference indexes the
// colour gradient as columns 4,5,6 of a 6-column array
// (jaxutil/tetra_quad.py:196-199 with utils/compare_quad.py:129), which after
// JAX's index clamping reads (gy, gz, gz).  grd_mode = 0 uses columns 3,4,5
// (gx, gy, gz), which is what the rasterizer integrates; grd_mode = 1
// reproduces the reference's indexing.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {
struct D3 {
  double x, y, z;
};
inline D3 sub(D3 a, D3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
inline double dot(D3 a, D3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
inline D3 cross(D3 a, D3 b) { return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x}; }
inline int sgn(double v) { return (v > 0) - (v < 0); }
// jaxutil/tetra_quad.py:101-115
inline bool same_side(D3 v1, D3 v2, D3 v3, D3 v4, D3 p) {
  D3 n = cross(sub(v2, v1), sub(v3, v1));
  return sgn(dot(n, sub(v4, v1))) * sgn(dot(n, sub(p, v1))) > 0;
}
// jaxutil/tetra_quad.py:117-133
inline bool point_in_tet(const D3 v[4], D3 p) {
  return same_side(v[0], v[1], v[2], v[3], p) && same_side(v[1], v[2], v[3], v[0], p) &&
         same_side(v[2], v[3], v[0], v[1], p) && same_side(v[3], v[0], v[1], v[2], p);
}

// 4x4 inverse of a rigid [R|t] world->camera matrix is not assumed; general
// Gauss-Jordan so that cam_pos = inv(viewmat)[:3,3] (jaxutil/tetra_quad.py:279).
inline bool inv4(const double* m, double* out) {
  double a[4][8];
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      a[i][j] = m[4 * i + j];
      a[i][4 + j] = i == j;
    }
  for (int c = 0; c < 4; ++c) {
    int piv = c;
    for (int r = c + 1; r < 4; ++r)
      if (std::fabs(a[r][c]) > std::fabs(a[piv][c])) piv = r;
    if (a[piv][c] == 0) return false;
    for (int j = 0; j < 8; ++j) std::swap(a[c][j], a[piv][j]);
    double s = a[c][c];
    for (int j = 0; j < 8; ++j) a[c][j] /= s;
    for (int r = 0; r < 4; ++r)
      if (r != c) {
        double f = a[r][c];
        for (int j = 0; j < 8; ++j) a[r][j] -= f * a[c][j];
      }
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) out[4 * i + j] = a[i][4 + j];
  return true;
}
}  // namespace

extern "C" {

// Renders pixels [pix0, pix1) (row-major index y*width+x) of the image.
// vertex_color is [T,6] = cell_values[:,1:], tet_density is [T]
// (utils/compare_quad.py:129-136).  out is [pix1-pix0, 5] = (r, g, b, alpha,
// distortion).  If g_density / g_color are non-null they receive the gradient
// of sum(rgb) over the rendered pixels (utils/compare_quad.py:164-184; the
// vertex gradient of the quadrature is identically zero and is not produced).
int quad_render(const float* vertices, int64_t V, const int32_t* indices, int64_t T, const float* vertex_color,
                const float* tet_density, int height, int width, const float* viewmat, float fx, float fy,
                float tmin, int n_samples, int64_t pix0, int64_t pix1, int grd_mode, float* out, double* g_density,
                double* g_color, int nthreads) {
  double vm[16], inv[16];
  for (int i = 0; i < 16; ++i) vm[i] = viewmat[i];
  if (!inv4(vm, inv)) return 1;
  D3 cam = {inv[3], inv[7], inv[11]};
  // tdist: jaxutil/tetra_quad.py:283-291
  double zmin = 1e300, zmax = -1e300;
  for (int64_t i = 0; i < V; ++i) {
    double z = vm[8] * vertices[3 * i] + vm[9] * vertices[3 * i + 1] + vm[10] * vertices[3 * i + 2] + vm[11];
    zmin = std::min(zmin, z);
    zmax = std::max(zmax, z);
  }
  double start = std::max(zmin, (double)tmin), end = zmax * 1.2;
  const int S = n_samples - 1;  // intervals
  std::vector<double> tdist(n_samples);
  for (int i = 0; i < n_samples; ++i) tdist[i] = (end - start) * (double(i) / double(n_samples - 1)) + start;
  std::vector<D3> tv((size_t)T * 4);
  for (int64_t t = 0; t < T; ++t)
    for (int k = 0; k < 4; ++k) {
      int64_t vi = indices[4 * t + k];
      tv[4 * t + k] = {vertices[3 * vi], vertices[3 * vi + 1], vertices[3 * vi + 2]};
    }
  const int gi[2][3] = {{3, 4, 5}, {4, 5, 5}};
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
  const bool want_grad = g_density && g_color;
#pragma omp parallel
  {
    std::vector<double> dens(S), col(3 * (size_t)S), wts(S), accs(S);
    std::vector<std::vector<int32_t>> inside(want_grad ? S : 0);
    std::vector<double> ld(want_grad ? (size_t)T : 0), lc(want_grad ? (size_t)T * 6 : 0);
#pragma omp for schedule(dynamic, 1)
    for (int64_t p = pix0; p < pix1; ++p) {
      int y = int(p / width), x = int(p % width);
      // rays: jaxutil/tetra_quad.py:253-273
      double dx = (x + 0.5 - width / 2.0) / fx, dy = (y + 0.5 - height / 2.0) / fy, dz = 1.0;
      double nrm = std::sqrt(dx * dx + dy * dy + dz * dz);
      dx /= nrm; dy /= nrm; dz /= nrm;
      D3 d = {vm[0] * dx + vm[4] * dy + vm[8] * dz, vm[1] * dx + vm[5] * dy + vm[9] * dz,
              vm[2] * dx + vm[6] * dy + vm[10] * dz};
      std::fill(dens.begin(), dens.end(), 0.0);
      std::fill(col.begin(), col.end(), 0.0);
      if (want_grad)
        for (auto& v : inside) v.clear();
      // query: jaxutil/tetra_quad.py:142-224
      for (int64_t t = 0; t < T; ++t) {
        const D3* v = &tv[4 * t];
        double td = tet_density[t];
        const float* vc = vertex_color + 6 * t;
        for (int s = 0; s < S; ++s) {
          double tm = 0.5 * (tdist[s] + tdist[s + 1]);
          D3 q = {cam.x + d.x * tm, cam.y + d.y * tm, cam.z + d.z * tm};
          if (!point_in_tet(v, q)) continue;
          D3 c = sub(q, v[0]);
          double off = vc[gi[grd_mode][0]] * c.x + vc[gi[grd_mode][1]] * c.y + vc[gi[grd_mode][2]] * c.z;
          dens[s] += td;
          col[3 * s + 0] += (vc[0] + off) * td;
          col[3 * s + 1] += (vc[1] + off) * td;
          col[3 * s + 2] += (vc[2] + off) * td;
          if (want_grad) inside[s].push_back((int32_t)t);
        }
      }
      // weights: jaxutil/tetra_quad.py:58-72,74-99
      double acc = 0, rgb[3] = {0, 0, 0}, alpha = 0;
      for (int s = 0; s < S; ++s) {
        double dd = dens[s] * (tdist[s + 1] - tdist[s]);
        double om = -std::expm1(-dd);
        double w = om * std::exp(-acc);  // exp(log(1 - exp(-dd)) + log_trans)
        wts[s] = w;
        accs[s] = acc;
        acc += dd;
        alpha += w;
        if (dens[s] > 1e-6)
          for (int k = 0; k < 3; ++k) rgb[k] += w * col[3 * s + k] / dens[s];
      }
      // distortion: jaxutil/tetra_quad.py:35-48, with mass = total density
      double msum = 0;
      for (int s = 0; s < S; ++s) msum += dens[s];
      double mclip = std::max(msum, 1e-8);
      double inter = 0, intra = 0, pw = 0, pwu = 0;
      for (int s = 0; s < S; ++s) {
        double w = dens[s] / mclip, u = 0.5 * (tdist[s] + tdist[s + 1]);
        inter += 2.0 * w * (u * pw - pwu);  // sum over ordered pairs, both orders
        pw += w;
        pwu += w * u;
        intra += w * w * (tdist[s + 1] - tdist[s]);
      }
      float* o = out + 5 * (p - pix0);
      o[0] = float(rgb[0]); o[1] = float(rgb[1]); o[2] = float(rgb[2]); o[3] = float(alpha);
      o[4] = float(inter + intra / 3.0);
      if (want_grad) {
        // d sum(rgb) / d density_t and / d vertex_color_t, by reverse accumulation.
        // rgb_k = sum_s w_s C_sk / D_s,  w_s = (1-exp(-D_s dl_s)) exp(-sum_{s'<s} D_s' dl_s')
        std::fill(ld.begin(), ld.end(), 0.0);
        std::fill(lc.begin(), lc.end(), 0.0);
        double suffix = 0;  // sum_{s' > s} w_s' * (sum_k colour_s'k)
        for (int s = S - 1; s >= 0; --s) {
          double dl = tdist[s + 1] - tdist[s];
          double csum = 0;
          if (dens[s] > 1e-6) csum = (col[3 * s] + col[3 * s + 1] + col[3 * s + 2]) / dens[s];
          double dd = dens[s] * dl;
          // gradient wrt D_s: own weight term + attenuation of later samples
          double trans_s = std::exp(-accs[s]);  // transmittance in front of sample s
          double g_D = dl * std::exp(-dd) * trans_s * csum - dl * suffix;
          double g_C = dens[s] > 1e-6 ? wts[s] / dens[s] : 0.0;  // wrt each C_sk
          if (dens[s] > 1e-6) g_D += -wts[s] * csum / dens[s];
          double tm = 0.5 * (tdist[s] + tdist[s + 1]);
          D3 q = {cam.x + d.x * tm, cam.y + d.y * tm, cam.z + d.z * tm};
          for (int32_t t : inside[s]) {
            const float* vc = vertex_color + 6 * t;
            D3 c = sub(q, tv[4 * (size_t)t]);
            double off = vc[gi[grd_mode][0]] * c.x + vc[gi[grd_mode][1]] * c.y + vc[gi[grd_mode][2]] * c.z;
            double td = tet_density[t];
            // D_s = sum td ; C_sk = sum (vc_k + off) td
            ld[t] += g_D + g_C * ((vc[0] + off) + (vc[1] + off) + (vc[2] + off));
            for (int k = 0; k < 3; ++k) lc[6 * (size_t)t + k] += g_C * td;
            double cc[3] = {c.x, c.y, c.z};
            for (int k = 0; k < 3; ++k) lc[6 * (size_t)t + gi[grd_mode][k]] += 3.0 * g_C * td * cc[k];
          }
          suffix += wts[s] * csum;
        }
#pragma omp critical
        {
          for (int64_t t = 0; t < T; ++t) {
            g_density[t] += ld[t];
            for (int k = 0; k < 6; ++k) g_color[6 * t + k] += lc[6 * (size_t)t + k];
          }
        }
      }
    }
  }
  return 0;
}

}  // extern "C"
