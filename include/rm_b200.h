/*
 * rm_b200 — C ABI of the B200 (sm_100a) differentiable tetrahedral tile rasterizer.
 *
 * Drop-in boundary for the hot path of half-potato/radiance_meshes'
 * delaunay_rasterization package.  Every entry point takes raw device
 * pointers, explicit sizes and a CUDA stream; nothing here allocates or frees
 * device memory (the caller owns outputs and workspaces), nothing keeps global
 * mutable state unless an entry point says otherwise, and all work is
 * stream-ordered on the stream passed in.  Return value: 0 on success, a
 * negative RM_ERR_* code for host-detected errors (see rm_strerror).
 * Device-detected conditions are reported through RmBinInfo.status.
 *
 * Citations are paths inside the reference project.
 */
#ifndef RM_B200_H_
#define RM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RM_OK 0
#define RM_ERR_INVALID_ARG (-1)
#define RM_ERR_CUDA (-2)
#define RM_ERR_TOO_MANY_KEYS (-3)
#define RM_ERR_WORKSPACE (-4)
#define RM_ERR_STATIC_SCRATCH (-5)

/* bits of RmBinInfo.status */
#define RM_STATUS_NAN_VERTEX 1u   /* a vertex coordinate is NaN (tile_shader_slang.py:78 asserts on this) */
#define RM_STATUS_KEY_OVERFLOW 2u /* more than 2^31-1 (tile, tet) pairs (int32 cumsum, tile_shader_slang.py:36) */
#define RM_STATUS_BAD_INDEX 4u    /* a tet names a vertex outside [0, n_vertices): the tet is treated as culled
                                     (the reference would read out of bounds) */

/* Floats per packed tet record (24 used by the integration + 12 for the hull edge
 * lines of the projected tet, used to cull whole tiles) and per record-gradient row. */
#define RM_RECORD_FLOATS 36
#define RM_GRAD_RECORD_FLOATS 24

/*
 * Camera, the reference's `tcam` dictionary (data/camera.py:72-91 plus the tile
 * fields of utils/train_util.py:30-37; device-side view slang/camera.slang:13-29).
 * The four arrays are DEVICE pointers exactly as the reference passes them
 * (small CUDA tensors), so building this struct needs no host synchronisation.
 */
typedef struct RmCamera {
  const float* world_view_transform; /* [4,4] row-major world->camera */
  const float* K;                    /* [3,3] */
  const float* cam_pos;              /* [3] */
  const float* distortion_params;    /* [4] k1 k2 p1 p2 */
  int32_t image_height, image_width;
  int32_t camera_type;               /* 0 perspective, 1 fisheye */
  float fovy, fovx, min_t;
  int32_t tile_height, tile_width, grid_height, grid_width;
  /* Screen-tile band [tile_row_begin, tile_row_end) this call is restricted to;
   * 0, grid_height for the whole frame.  No counterpart in the reference (it is
   * single-GPU); used to split one frame over several GPUs by tile rows. */
  int32_t tile_row_begin, tile_row_end;
} RmCamera;

/* Written by rm_project_and_bin at the start of the info buffer (device memory). */
typedef struct RmBinInfo {
  int64_t n_keys;        /* N = sum of tiles_touched */
  int64_t n_region_keys; /* sum over tets of the 8 x 4-tile regions their rectangle touches */
  int32_t n_visible;     /* tets with tiles_touched > 0 */
  uint32_t status;       /* RM_STATUS_* bits */
} RmBinInfo;

/*
 * Hit lists, written by rm_forward and walked by rm_backward (device pointers).  No
 * counterpart in the reference, whose backward pass walks every tile list again and
 * repeats every intersection test.  A unit is one group of 16 pixels of a tile (tile t,
 * group s of S = ceil(tile_width*tile_height / 16): unit t*S + s).  The forward pass
 * evaluates a unit's list in batches of 16 entries that can cover one of its pixels (the
 * last batch may hold fewer) and records every batch, in list order:
 *   counts[G*S] i32        number of recorded entries of the unit
 *   ids[N*S] i32           their tet ids, unit (t, s) at [start(t)*S + s*len(t), ... + counts)
 *   masks[N*S + 16*G*S] u16  for batch b of unit q = t*S + s, at [start(t)*S + s*len(t) + 16*q + 16*b, + 16):
 *                          per pixel of the group, the bit set of the batch entries the pixel
 *                          hit with positive optical depth while still active (bit = entry
 *                          index inside the batch)
 *   tet_flags[T] u8        set to 1 for every tet that appears in some hit list; the caller
 *                          zero-fills it before rm_forward.  The backward pass clears and reads
 *                          the record-gradient rows of flagged tets only.
 * with start/len from tile_ranges.  Slots beyond a unit's count are left unwritten.
 */
typedef struct RmHitList {
  int32_t* counts;
  int32_t* ids;
  uint16_t* masks;
  uint8_t* tet_flags;
} RmHitList;

const char* rm_strerror(int code);
int rm_version(void);

/* Bytes of workspace rm_project_and_bin needs for T tets and G = grid_height*grid_width tiles. */
size_t rm_bin_workspace_bytes(int64_t n_tets, int64_t n_tiles);

/*
 * Stage 1 + the size-independent half of stages 2-4.
 * Replaces VertexShader.forward / vertex_shader (tile_shader_slang.py:77-125,
 * slang/vertex_shader.slang:20-89), torch.cumsum (tile_shader_slang.py:36) and
 * compute_tile_ranges (slang/tile_shader.slang:99-125).
 *   indices[T,4] i32, vertices[V,3] f32 ->
 *   tiles_touched[T] i32, rect_tile_space[T,4] i32, vs_tetra[T,3] f32 (column 2 =
 *   clamped circumsphere power, the sort depth), circumcenter[T,3] f32 (zeros for
 *   culled tets), tile_ranges[G,2] i32 (start,end of each tile's list; (0,0) if
 *   empty), info (RmBinInfo).  Every output element is written.
 * workspace must hold rm_bin_workspace_bytes(T, G) bytes, 256-byte aligned, and
 * must stay untouched until rm_build_tile_lists has consumed it.
 */
int rm_project_and_bin(const int32_t* indices, int64_t n_tets, const float* vertices, int64_t n_vertices,
                       const RmCamera* cam, int32_t* tiles_touched, int32_t* rect_tile_space, float* vs_tetra,
                       float* circumcenter, int32_t* tile_ranges, RmBinInfo* info, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Bytes of scratch rm_build_tile_lists needs for n_region_keys (region, tet) pairs on a
 * grid_height x grid_width tile grid (0 if the grid has more than 2^22 regions of 8 x 4
 * tiles, which is not supported). */
size_t rm_list_scratch_bytes(int64_t n_region_keys, int grid_height, int grid_width);

/*
 * Stages 2-3: per-tile tet lists ordered by (sort depth bits, tet id).
 * Replaces generate_keys (slang/tile_shader.slang:49-97) + sort_by_keys
 * (sort_by_keys/sort_by_keys.cu:9-53): the result equals the value array of a
 * stable ascending sort of the keys (tile << 32 | sortable(depth)).
 *   n_keys and n_region_keys must be RmBinInfo.n_keys and .n_region_keys read back
 *   by the caller; sorted_tetra_idx[N] i32 out; scratch:
 *   rm_list_scratch_bytes(n_region_keys, grid_height, grid_width) bytes, 256-byte
 *   aligned, caller-provided.
 */
int rm_build_tile_lists(const int32_t* rect_tile_space, const int32_t* tile_ranges, int64_t n_tets,
                        const RmCamera* cam, int64_t n_keys, int64_t n_region_keys, void* workspace, void* scratch,
                        size_t scratch_bytes, int32_t* sorted_tetra_idx, void* stream);

/*
 * Per-frame packed tet records (4 outward face planes relative to the camera
 * position, colour field, density, and the edge lines of the projected hull in pixel
 * coordinates): the staged form of load_tet_alphablend_interp
 * (slang/interp_version.slang:100-153).
 * tiles_touched may be NULL (pack every tet) or [T] (skip culled tets).
 * records[T, RM_RECORD_FLOATS] f32 out, 16-byte aligned; with tiles_touched given, the rows of
 * culled tets (which appear in no tile list) are left unwritten.  A tet that names a vertex
 * outside [0, n_vertices) gets a record that no pixel can hit.
 */
int rm_pack_records(const int32_t* indices, const float* vertices, const float* cell_values, int64_t n_tets,
                    int64_t n_vertices, const RmCamera* cam, const int32_t* tiles_touched, float* records,
                    void* stream);

/*
 * Forward integration.  Replaces splat_tiled (slang/alphablend_shader_interp.slang:371-431,
 * host side alphablend_tiled_slang_interp.py:11-52).
 *   ray_jitter[H,W,2] f32 -> output_img[H,W,4] (r,g,b,log-transmittance),
 *   distortion_img[H,W,5], n_contributors[H,W] i32.  Every pixel of the band is written.
 *   hits (optional, may be NULL): hit lists for rm_backward, see RmHitList.
 */
int rm_forward(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
               const RmCamera* cam, const float* ray_jitter, float* output_img, float* distortion_img,
               int32_t* n_contributors, const RmHitList* hits, void* stream);

/*
 * Forward pass of the constant-colour debug renderer.  Replaces splat_tiled of
 * slang/alphablend_shader.slang:279-330 (alpha_blend :100-182, evaluate_tetra
 * utils.slang:160-186; host side alphablend_tiled_slang.py:83-128), forward only.
 *   records: rm_pack_records of cell values (density, r, g, b, 0, 0, 0);
 *   samples at the pixel centres; output_img[H,W,4] = (r, g, b, transmittance),
 *   distortion_img[H,W,4], n_contributors[H,W]; a pixel stops once its transmittance
 *   is below 1/255.  ladder_p must not be 0.
 */
int rm_forward_constant_color(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                              const RmCamera* cam, float pre_multi, float ladder_p, float* output_img,
                              float* distortion_img, int32_t* n_contributors, void* stream);

/*
 * Backward pass of the constant-colour debug renderer.  Replaces splat_tiled.bwd / bwd_alpha_blend of
 * slang/alphablend_shader.slang:186-277 (host side alphablend_tiled_slang.py:131-192), with the reference's
 * formulation: pairs with alpha < 1/255 skipped, the state in front of a tet recovered by undoing the update.
 *   records and cell_values: as passed to rm_forward_constant_color (cell values (density, r, g, b, 0, 0, 0));
 *   output_img, distortion_img, n_contributors: what that call wrote; grad_distortion_img[H,W,4];
 *   grad_records[T, RM_GRAD_RECORD_FLOATS] and tet_flags[T] are caller-provided scratch (filled here);
 *   vertices_grad[V,3] and cell_values_grad[T,7] = gradients of (density, r, g, b, -, -, -) are fully written.
 */
int rm_backward_constant_color(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                               const RmCamera* cam, float pre_multi, float ladder_p, const float* output_img,
                               const float* distortion_img, const int32_t* n_contributors,
                               const float* grad_output_img, const float* grad_distortion_img, const int32_t* indices,
                               const float* vertices, const float* cell_values, int64_t n_tets, int64_t n_vertices,
                               float* grad_records, uint8_t* tet_flags, float* vertices_grad, float* cell_values_grad,
                               void* stream);

/*
 * Backward integration.  Replaces splat_tiled.bwd / bwd_alpha_blend
 * (slang/alphablend_shader_interp.slang:273-369, host side
 * alphablend_tiled_slang_interp.py:70-112).
 *   hits are the hit lists rm_forward wrote for the same lists and inputs (sorted_tetra_idx and
 *   n_contributors are accepted for symmetry with the reference's call and not read);
 *   grad_records[T, RM_GRAD_RECORD_FLOATS] is caller-provided scratch (the rows of flagged tets are
 *   zeroed here; the others are neither written nor read);
 *   vertices_grad[V,3] and cell_values_grad[T,7] are fully written (zeroed here first).
 */
int rm_backward(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                const RmCamera* cam, const float* ray_jitter, const float* output_img,
                const float* distortion_img, const int32_t* n_contributors, const RmHitList* hits,
                const float* grad_output_img, const float* grad_distortion_img, const int32_t* indices,
                const float* vertices, const float* cell_values, int64_t n_tets, int64_t n_vertices,
                float* grad_records, float* vertices_grad, float* cell_values_grad, void* stream);

/*
 * The two halves of rm_backward, for callers that want to start work on finished gradients early (a
 * multi-GPU job sums the cell-value gradients of one range of tets over the ranks while the next
 * range is still being finished).  No counterpart in the reference, which is single-GPU.
 *   rm_backward_integrate: zeroes vertices_grad, clears the record-gradient rows of flagged tets and
 *     accumulates the record gradients of the whole frame (the pixel walk).
 *   rm_backward_finish: the per-tet chain rule for tets [tet_begin, tet_end): writes rows
 *     [tet_begin, tet_end) of cell_values_grad[T,7] and adds to vertices_grad[V,3], which is complete
 *     once every tet has been finished.  Ranges whose begin is a multiple of 256 keep the stores wide.
 * rm_backward is rm_backward_integrate followed by rm_backward_finish(0, n_tets).
 */
int rm_backward_integrate(const int32_t* tile_ranges, const float* records, const RmCamera* cam,
                          const float* ray_jitter, const float* output_img, const float* distortion_img,
                          const RmHitList* hits, const float* grad_output_img, const float* grad_distortion_img,
                          int64_t n_tets, int64_t n_vertices, float* grad_records, float* vertices_grad, void* stream);
int rm_backward_finish(const int32_t* indices, const float* vertices, const float* cell_values, int64_t tet_begin,
                       int64_t tet_end, int64_t n_tets, const RmCamera* cam, const float* grad_records,
                       const RmHitList* hits, float* vertices_grad, float* cell_values_grad, void* stream);

/*
 * Feature activation of a frozen model, the step before the rasterizer on the
 * rendering path.  Replaces activate_output (utils/model_util.py:93-105, with
 * offset_normalize :81-91 and eval_sh utils/eval_sh_py.py:121-179; callers
 * tile_benchmark.py:62-67, models/frozen.py:216-223), forward only:
 *   density[T], rgb[T,3], grd[T,3] f32, sh[T, n_sh_rest, 3] f32 or f16 (coefficients
 *   beyond degree 0; (sh_degree+1)^2-1 <= n_sh_rest <= 24), indices[T,4] i32, circumcenters[T,3], vertices[V,3],
 *   camera_center[3] (device) -> features[T,7] = (density, softplus_10(SH colour at
 *   vertex 0), colour gradient scaled by min(rgb) / circumradius).
 */
int rm_activate_output(const float* camera_center, const float* density, const float* rgb, const float* grd,
                       const void* sh, int sh_is_half, const int32_t* indices, const float* circumcenters,
                       const float* vertices, int64_t n_tets, int sh_degree, int n_sh_rest, float* features,
                       void* stream);

/*
 * Densification statistics.  Replaces calc_tet_err (slang/alphablend_shader_interp.slang:433-599,
 * host side internal/render_err.py:119-150): every pixel walks its tile list from the
 * pixel centre and every hit adds its weight T (transmittance in front of the tet times
 * the tet's optical depth, with the reference's initial log-transmittance of 1) times
 * (1, err, err^2, -, -, ssim, entry point xyz, exit point xyz, 1, mid point xyz) to
 * tet_err[T,16] and (1, max int(65535*T)) to tet_count[T,2].  Both outputs are zeroed here.
 *   pixel_err[H,W], ssim_err[H,W] f32; records from rm_pack_records.
 */
int rm_tet_err(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
               const RmCamera* cam, const float* pixel_err, const float* ssim_err, int64_t n_tets, float* tet_err,
               int32_t* tet_count, void* stream);

/*
 * Reverse of stage 1 with respect to the vertices.  Replaces vertex_shader.bwd
 * (tile_shader_slang.py:128-150).  grad_vs_tetra[T,3] (only column 2 is read)
 * and grad_circumcenter[T,3] -> vertices_grad[V,3], zeroed here first.
 */
int rm_vertex_backward(const int32_t* indices, const float* vertices, int64_t n_tets, int64_t n_vertices,
                       const RmCamera* cam, const int32_t* tiles_touched, const float* grad_vs_tetra,
                       const float* grad_circumcenter, float* vertices_grad, void* stream);

/*
 * Backward integration without any caller-provided or allocated scratch.
 * No counterpart in the reference.
 *
 * Some hosts of this library cannot allocate device memory at the point where
 * the backward pass runs: a plugin that is handed fixed input/output buffers by
 * an engine that owns the allocator, code running under a memory budget that was
 * fixed before the frame, or a callback in which cudaMalloc is forbidden.  This
 * variant of rm_backward takes the same inputs and outputs but keeps its one
 * scratch buffer (the per-tet record-gradient rows, RM_GRAD_RECORD_FLOATS floats per
 * tet) in a static device array inside the library, RM_STATIC_SCRATCH_MAX_TETS
 * rows = 12 MiB, which every GPU that loads the library holds until the process
 * exits.  It calls no cudaMalloc/cudaFree or other allocating routine.
 *
 *   - n_tets > RM_STATIC_SCRATCH_MAX_TETS is rejected with RM_ERR_STATIC_SCRATCH.
 *   - The first call on each device looks up the array's device address; make
 *     that first call outside any stream capture.
 *   - All calls on a device share the array.  Each call clears the rows it
 *     uses, but two calls whose kernels overlap on the GPU (different streams)
 *     race on it: serialise them.
 * Results equal rm_backward's up to the order of floating-point atomics.
 */
#define RM_STATIC_SCRATCH_MAX_TETS 131072
int rm_backward_static_scratch(const int32_t* sorted_tetra_idx, const int32_t* tile_ranges, const float* records,
                               const RmCamera* cam, const float* ray_jitter, const float* output_img,
                               const float* distortion_img, const int32_t* n_contributors,
                               const RmHitList* hits, const float* grad_output_img,
                               const float* grad_distortion_img,
                               const int32_t* indices, const float* vertices, const float* cell_values,
                               int64_t n_tets, int64_t n_vertices, float* vertices_grad, float* cell_values_grad,
                               void* stream);

/*
 * Sum of floats [float_begin, float_end) of a buffer over the `world` GPUs of one NVSwitch domain,
 * in place on every GPU, for multi-GPU jobs that render one view per GPU and sum the gradients (no
 * counterpart in the reference, which is single-GPU).  `multicast_buffer` is the NVLink MULTICAST
 * address of the buffer: every rank holds the buffer at the same offset of a symmetric allocation
 * bound to one multicast object (e.g. torch.distributed._symmetric_memory: empty(), rendezvous(),
 * multicast_ptr).  Rank `rank` launches one kernel that pulls the sum of its 1/world slice through
 * the switch (multimem.ld_reduce) and stores it to all GPUs (multimem.st).  Both bounds must be
 * multiples of 4 floats and the address 16-byte aligned.  The kernel waits for nothing; the caller
 * orders it on `stream`: a barrier among the ranks after the last write to the range and before this
 * call, and another after it before any rank reads the sums.
 */
int rm_multimem_sum(float* multicast_buffer, int64_t float_begin, int64_t float_end, int rank, int world,
                    void* stream);

/*
 * Optional per-kernel timing, a measurement aid with no counterpart in the
 * reference (which only has commented-out wall-clock prints,
 * alphablend_tiled_slang.py:39-40).  While enabled, every kernel launch of the
 * entry points above is bracketed by a CUDA event pair on its stream; this is
 * process-global state.  rm_profile_read waits for the recorded events, writes
 * up to max_records durations (milliseconds) to ms and the matching
 * newline-separated kernel names to names, clears the records and returns how
 * many it wrote.
 */
void rm_profile_enable(int on);
int rm_profile_read(char* names, size_t names_bytes, float* ms, int max_records);

/* Number of kernels this library has launched in this process so far (all entry points, all
 * threads; memsets and copies are not kernels and are not counted).  A measurement aid with no
 * counterpart in the reference: the difference across a timed region is the number of this
 * library's launches inside it. */
int64_t rm_launch_count(void);

/*
 * Bounds-checked build of the library (compiled with -DRM_BOUNDS_CHECK; the tests' stand-in for a
 * memory checker, no counterpart in the reference).  In that build every index that depends on data
 * - list cursors, hit-list slots, ids read from lists and the rows they address - is compared with the
 * extent of its array before the access; a violation sets a bit of a status word and the access is
 * skipped, nothing traps.
 *   rm_debug_bounds_checked: 1 in the checked build, 0 otherwise (the other two are no-ops then).
 *   rm_debug_set_extent(which, n): extent of a caller-owned array of the integration stages, whose
 *     entry points carry no lengths: 0 list entries, 1 tets, 2 vertices, 3 hit-list id slots,
 *     4 hit-list mask slots, 5 hit-list units.
 *   rm_debug_bounds_status: waits for the device, returns the status word and clears it (bit = access
 *     site; 0 = every checked access was inside its array).
 */
int rm_debug_bounds_checked(void);
void rm_debug_set_extent(int which, int64_t n);
uint32_t rm_debug_bounds_status(void);

#ifdef __cplusplus
}
#endif
#endif /* RM_B200_H_ */
