/*
 * vetr.h — C ABI of the B200 (sm_100a) blending point rasterizer.
 *
 * This is the boundary a host program binds to: plain pointers and sizes, no C++ or tensor-library types.
 * Every function replaces a piece of the reference's rasterizer (lfranke/VET, src/lib/rendering); the comment
 * of each entry point cites what it stands in for.
 *
 * Conventions
 *   - All pointers named *device* pointers below must point to memory of the context's GPU.
 *   - Every call enqueues its work on the context's stream and returns without synchronising, unless stated.
 *   - Return value: VETR_OK (0) or a negative vetr_status.  Nothing aborts the process or traps the device.
 *     Conditions that can only be seen on the device (fragment buffer overflow) are recorded in a device
 *     status word that vetr_read_status() copies back.
 *   - A context is not thread-safe; distinct contexts are independent.  There is no process-global state.
 */
#ifndef VETR_H
#define VETR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VETR_MAX_LAYERS 5 /* RenderConstants.h:33 (max_layers) */
#define VETR_MAX_VIEWS 8  /* views handled by one launch; larger batches are processed in groups */

typedef enum vetr_status
{
    VETR_OK               = 0,
    VETR_E_INVALID_ARG    = -1,
    VETR_E_CUDA           = -2, /* a CUDA runtime call failed; vetr_last_cuda_error() has the code */
    VETR_E_UNSUPPORTED    = -3, /* camera model / option the library does not implement */
    VETR_E_LIST_OVERFLOW  = -4, /* more fragments than the fragment buffer holds (reported by vetr_read_status) */
    VETR_E_TOO_LARGE      = -5  /* a size exceeds a fixed limit of the entry point (vetr_read_status: a list longer than
                                   4096 fragments met the mode-2 backward pass, which skipped that pixel) */
} vetr_status;

/* Render modes: PointRendererCache::RenderMode, PointRenderer.h. */
#define VETR_MODE_FUZZY_DT 0
#define VETR_MODE_FULL_BLEND 1
#define VETR_MODE_FUZZY_BLEND 2
#define VETR_MODE_BILINEAR_BLEND 3

/* The RenderParams fields the kernels read: data/Settings.h:19-73, RenderConstants.h:36-60. */
typedef struct vetr_params
{
    int32_t render_mode;               /* VETR_MODE_* */
    int32_t num_layers;                /* 1..VETR_MAX_LAYERS */
    int32_t num_channels;              /* 3 or 4 (RenderBackward.cu:2474-2492) */
    int32_t drop_out_points_by_radius; /* bool */
    float   drop_out_radius_threshold; /* 0.6 */
    float   dist_cutoff;               /* 20 */
    int32_t use_environment_map;       /* bool: no background term */
    int32_t viewer_only;               /* bool: drop points whose confidence < stability_cutoff_value */
    float   stability_cutoff_value;
    int32_t debug_max_list_length;     /* <= 0: off */
    int32_t need_point_gradient;       /* bool */
    float   K_gradient_factor;         /* 0.5 */
    float   distortion_gradient_factor;/* 0.005 */
    float   output_background_mask_value;
    int32_t background_alpha_to_point0;/* bool, default 1: the reference adds the background entry's alpha
                                          gradient to descriptor 0's confidence gradient (RenderBackward.cu:1130,1157) */
    int32_t keep_sorted_lists;         /* bool: write the sorted lists back (needed by vetr_backward / vetr_get_lists) */
    float   depth_accept_blend;        /* 0.01: depth window of a fuzzy group, mode 2 (data/Settings.h:29) */
    float   depth_accept;              /* 0.01: relative depth window of the splat, mode 0 (data/Settings.h:28) */
    int32_t ghost_gradients;           /* bool, mode 0: position gradients from dropped-out points instead (Settings.h:31) */
} vetr_params;

/* ReducedImageInfo, data/SceneData.h:39-50. */
typedef struct vetr_view
{
    int32_t w, h;
    int32_t image_index;  /* row of poses_se3 */
    int32_t camera_index; /* row of intrinsics */
    int32_t camera_model; /* 0 = pinhole + distortion (the only model built) */
    float   crop[5];      /* crop_transform: fx fy cx cy s */
    float   rot[4];       /* crop_rotation, row-major 2x2 */
} vetr_view;

/* NeuralPointCloudCuda tensors, rendering/NeuralPointCloudCuda.h:81-106 (device pointers). */
typedef struct vetr_cloud
{
    const float*   position; /* [n,4] xyz + drop-out radius, 16-byte aligned */
    const int32_t* index;    /* [n]   point -> descriptor column */
    int32_t        n;
} vetr_cloud;

/* NeuralPointTexture tensors, models/NeuralTexture.h:114-126 (device pointers). */
typedef struct vetr_texture
{
    const float* texture;    /* [channels, n_tex] channel-major */
    const float* confidence; /* [n_tex] */
    const float* background; /* [channels] */
    int32_t      n_tex;
} vetr_texture;

/* PoseModule / IntrinsicsModule tensors, data/NeuralStructure.h:30-34,56-59 (device pointers). */
typedef struct vetr_cameras
{
    const double* poses_se3;  /* [n_img,8] world->camera: qx qy qz qw tx ty tz pad */
    const float*  intrinsics; /* [n_cam,13] fx fy cx cy s k1 k2 k3 k4 k5 k6 p1 p2 */
    int32_t       n_img, n_cam;
} vetr_cameras;

/*
 * Per-pixel fragment lists of one forward call: what the reference keeps in LayerCuda::counting /
 * scanned_counting / per_image_atomic_counters and in collections[b][l] (PointRenderer.h:66-110,
 * PointRenderer.cu:796-822).  All views and levels live in ONE pixel space of n_views * P entries
 * (P = pyramid pixels of a view; view-major, then level, then the banded order of VETR_PIXEL_BAND below) and ONE
 * fragment buffer.
 * Caller-owned device memory.
 */
typedef struct vetr_lists
{
    int32_t*  counts;   /* [n_views*P]  list length per pixel (P = vetr_pyramid_pixels) */
    int32_t*  ends;     /* [n_views*P]  end offset (exclusive) of the pixel's list in frags; its start is ends - counts */
    void*     frags;    /* [capacity] 32-byte fragment records, 32-byte aligned; ascending by key inside each list
                           after forward.  Record: uint64 key = depth bits << 32 | point index; float alpha
                           (confidence, or bilinear weight x confidence in mode 3); int32 descriptor index; float[4]
                           descriptor.  Everything the blend needs of a fragment sits in one 32-byte sector, so the
                           blend and the backward pass stream it instead of gathering through index -> descriptor. */
    int64_t   capacity; /* records in frags */
    int32_t*  status;   /* [4] device words: {total fragments F, overflow flag, longest list, number of work items} */
    int32_t*  items;    /* [items_capacity] work-item table written by the scan: first pixel of every run of pixels that
                           one thread block of the blend / backward kernels processes (balanced by fragments) */
    int64_t   items_capacity; /* >= vetr_item_table_entries(capacity, n_views*P) */
    uint8_t*  level_mask;  /* [n_views*n] written by vetr_forward when not NULL: bit l set = the point has a fragment on
                              pyramid level l of that view */
    float*    point_grad;  /* 16-byte aligned scratch of vetr_backward, indexed by (view, level, point): modes 1 and 2
                              [n_views*num_layers*n*2], the image-space gradient of the point's fragment on that level;
                              mode 3 [n_views*num_layers*n*4], the alpha gradient of its four bilinear fragments.  The
                              position / pose / intrinsics gradients (and mode 3's confidence gradient) are then formed
                              in one coalesced pass over the points: every fragment's term computed exactly as in
                              ProjectPointPinholeBackward, summed per point in a fixed order, no atomics on g_points.
                              Both arrays are required by vetr_backward in mode 3, and in modes 1 and 2 when
                              need_point_gradient is set; level_mask must be the one the forward call wrote.  Neither
                              needs initialising.  Mode 3 keeps a fragment's corner in the two top bits of the record's
                              descriptor index, so n_tex must stay below 2^30 there. */
    float*    pixel_scratch; /* [n_views*P*8] 16-byte aligned scratch of vetr_backward in modes 1-3: channel-interleaved
                                copies of out_color and grad_color over the pixel space (eight 16-byte loads fetch all
                                neighbour values of a fragment).  Needs no initialising. */
} vetr_lists;

typedef struct vetr_ctx vetr_ctx;

/* Creates a context on `device` that enqueues on `cuda_stream` (a cudaStream_t; NULL = the legacy default stream).
 * Replaces the process-global state of the reference (the __constant__ parameter blocks of RenderForward.cu:22-27 and
 * the cached PointRendererCache, PointRenderer.h:112-248). Allocates a few KB of device scratch; synchronous. */
int vetr_create(vetr_ctx** out, int device, void* cuda_stream);
void vetr_destroy(vetr_ctx* ctx);
int vetr_set_stream(vetr_ctx* ctx, void* cuda_stream);
const char* vetr_strerror(int status);
int vetr_last_cuda_error(const vetr_ctx* ctx);

/* Size of the pixel space of one w x h view with num_layers levels (successive integer halving, PointRenderer.cu:351-381):
 * the sum over the levels of w_l * (h_l rounded up to a multiple of VETR_PIXEL_BAND).  The pixel space orders the pixels
 * of a level in bands of VETR_PIXEL_BAND rows, column by column inside a band,
 *     offset(x, y) = (y / BAND) * BAND * w_l + BAND * x + y % BAND,
 * so that a run of consecutive pixels is a compact patch of the image and the fragments of neighbouring points land
 * near each other in the fragment buffer; the rows that pad the last band hold no fragments.  counts / ends of
 * vetr_lists are indexed like this; the images stay plain [view, channel, y, x] tensors. */
#define VETR_PIXEL_BAND 4
int64_t vetr_pyramid_pixels(int w, int h, int num_layers);

/* Entries the work-item table of vetr_lists needs for a fragment buffer of `capacity` records over `n_pixels_total` pixels. */
int64_t vetr_item_table_entries(int64_t capacity, int64_t n_pixels_total);

/* Upper bound of the number of fragments: n * num_layers * n_views (x4 in bilinear mode). */
int64_t vetr_max_fragments(int n_points, int n_views, const vetr_params* params);

/* Records the fragment buffer of vetr_lists must hold so that a call of n_views w x h views can never overflow: the
 * bound above in modes 1-3 (the reference sizes collections[b][l] after reading the counts back, PointRenderer.cu:796-822;
 * here nothing is read back); in mode 0, which keeps one accumulator record per pixel instead of lists, the size of the
 * pixel space, n_views * vetr_pyramid_pixels. */
int64_t vetr_list_capacity(int n_points, int n_views, int w, int h, const vetr_params* params);

/* Forward pass: CountingPrepassMulti + exclusive_scan + CollectMulti + SortMulti + BlendMulti / BlendMultiBilinear +
 * CreateMask for all views and levels (BlendPointCloudForward, PointRenderer.cu:657-1069).
 *   dropout    [n_views, n] float device array, 1 = point dropped (PointRenderer.cu:461-468), or NULL
 *   out_color  num_layers device pointers, level l is [n_views, channels, h_l, w_l]
 *   out_weight num_layers device pointers [n_views,1,h_l,w_l]: final transmittance (LayerCuda::weight), or NULL
 *   out_mask   num_layers device pointers [n_views,1,h_l,w_l] (CreateMask, PointRenderer.cu:216-235), or NULL
 *   out_depth  num_layers device pointers [n_views,1,h_l,w_l]: nearest depth, 100000 where empty (LayerCuda::depth), or NULL
 * n_views <= VETR_MAX_VIEWS; all views share w and h. */
int vetr_forward(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud, const vetr_texture* texture,
                 const vetr_cameras* cameras, const vetr_view* views, int n_views, const float* dropout,
                 const vetr_lists* lists, float* const* out_color, float* const* out_weight, float* const* out_mask,
                 float* const* out_depth);

/* Mode 0 (FUZZY_DT: DepthPrepassMulti, RenderForwardMulti, CombineAndFill, RenderForward.cu:180-406, PointRenderer.cu:24-52)
 * keeps no lists: vetr_forward uses lists->ends for the nearest depth of every pixel, lists->frags (capacity >= n_views*P)
 * as accumulators and leaves the number of accepted points of every pixel in lists->counts; out_weight is that number.
 *
 * Backward pass of the forward call that filled `lists`: BlendBackwards2 / BlendBackwardsBilinear for all views and
 * levels (BlendPointCloudBackward, PointRenderer.cu:1111-1250; kernels RenderBackward.cu:1083-1513, 2893-3232).
 * (mode 0: CombineAndFillBackward + RenderBackward, RenderBackward.cu:27-76, 131-474; `dropout` must be the mask given to
 * vetr_forward, other modes ignore it).
 * Gradients are ADDED to the caller's buffers as raw sums (the caller zero-fills; several calls may accumulate):
 *   g_desc     [n_tex,4] point-major descriptor gradient (columns >= channels stay untouched)
 *   g_conf     [n_tex]
 *   g_points   [n,4] xyz gradient sum + hit count in .w, or NULL (out_gradient_points + out_gradient_points_count)
 *   g_background [channels]
 *   g_pose     [n_img,6] double, g_pose_count [n_img] float, or NULL
 *   g_intr     [n_cam,13] float, g_intr_count [n_cam] float, or NULL
 * out_color are the images the forward call wrote; grad_color their gradients (same shapes). */
int vetr_backward(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud, const vetr_texture* texture,
                  const vetr_cameras* cameras, const vetr_view* views, int n_views, const float* dropout, const vetr_lists* lists,
                  const float* const* out_color, const float* const* grad_color, float* g_desc, float* g_conf,
                  float* g_points, float* g_background, double* g_pose, float* g_pose_count, float* g_intr,
                  float* g_intr_count);

/* The same in two calls, for hosts that start exchanging the descriptor / confidence gradients while the position
 * gradients are still being formed: VETR_BACKWARD_FRAGMENTS enqueues the per-fragment kernels (afterwards g_desc,
 * g_background and, in modes 1 and 2, g_conf are final), VETR_BACKWARD_POINTS the per-point pass (g_points, g_pose,
 * g_intr; in mode 3 also g_conf).  vetr_backward is both.  Mode 0 does everything in the first phase. */
#define VETR_BACKWARD_FRAGMENTS 1
#define VETR_BACKWARD_POINTS 2
int vetr_backward_phase(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud, const vetr_texture* texture,
                        const vetr_cameras* cameras, const vetr_view* views, int n_views, const float* dropout,
                        const vetr_lists* lists, const float* const* out_color, const float* const* grad_color,
                        float* g_desc, float* g_conf, float* g_points, float* g_background, double* g_pose,
                        float* g_pose_count, float* g_intr, float* g_intr_count, int phases);

/* Epilogue of the backward pass: converts the accumulation buffers into the tensors the reference returns
 * (PointRenderer.cu:1251-1322): g_texture [channels,n_tex] channel-major (transpose of g_desc), and the count
 * normalisation of NormalizeGradient / NormalizeGradientDevTensor (PointRenderer.cu:1072-1109): point gradients
 * [n,4] divided by their hit count (.w is set to 0 afterwards, counts are written to g_points_count [n] if given),
 * pose and intrinsics gradients divided by their counts.  Any pointer may be NULL to skip that part. */
int vetr_finalize_gradients(vetr_ctx* ctx, int channels, int n_tex, const float* g_desc, float* g_texture, int n,
                            float* g_points, float* g_points_count, int n_img, double* g_pose,
                            const float* g_pose_count, int n_cam, float* g_intr, const float* g_intr_count);

/* View-sharded training on several GPUs of one node (the reference is single-GPU; this has no counterpart there).
 * Every rank keeps its raw gradient sums of a step in ONE buffer, [descriptor gradient n_tex*4 | position gradient +
 * hit count n*4 | confidence gradient n_tex] floats (vetr_exchange_raw_floats), in memory its peers can address
 * (CUDA peer access: IPC or VMM mappings; torch's symmetric memory gives such pointers).  vetr_exchange_finalize is
 * the sum over the ranks and vetr_finalize_gradients in one kernel over that peer memory: the rank reduces its 1/world
 * slice of every rank's raw buffer and stores the finished slice (texture gradient [channels, n_tex], position
 * gradient [n,4] averaged by hit count, confidence gradient [n_tex]; vetr_exchange_out_floats, position segment at
 * channels*n_tex rounded up to 4 floats) into every rank's output buffer.  It moves the bytes of a reduce-scatter plus
 * an all-gather and replaces NCCL all-reduce + the epilogue kernels.
 * Ordering is the caller's: the kernel must start after the backward kernels of ALL ranks have finished and its
 * outputs may be read after the exchange kernels of ALL ranks have finished - enqueue a collective on the same stream
 * before and after it (the all-reduce of the pose gradients and of their counts serve).  The kernel itself waits on
 * nothing.  world = 1 is allowed (a local epilogue). */
#define VETR_MAX_RANKS 16
typedef struct vetr_exchange
{
    int32_t rank, world;
    const float* raw[VETR_MAX_RANKS]; /* raw[k]: rank k's raw buffer as seen from this rank, 16-byte aligned */
    float*       out[VETR_MAX_RANKS]; /* out[k]: rank k's output buffer as seen from this rank, 16-byte aligned */
    const float* raw_multicast;       /* optional: address of the NVSwitch multicast object bound to all ranks' raw buffers */
    float*       out_multicast;       /* (and output buffers).  Both or neither.  When given, the sum is done by the switch
                                         (multimem.ld_reduce) and the results are stored to all ranks at once (multimem.st):
                                         the rank moves 1/world of the bytes.  fp32 sums in the switch's order. */
} vetr_exchange;
int64_t vetr_exchange_raw_floats(int n_tex, int n);
int64_t vetr_exchange_out_floats(int channels, int n_tex, int n);
int vetr_exchange_finalize(vetr_ctx* ctx, const vetr_exchange* ex, int channels, int n_tex, int n);
/* One or two of the three segments only (VETR_SEG_* bits), on a grid of ctas_per_sm (1..8) thread blocks per SM: lets a
 * host run the descriptor / confidence part on a second stream beside vetr_backward_phase(VETR_BACKWARD_POINTS), with a
 * small grid so that both kernels are resident, and the position part afterwards.  Each part needs the ordering
 * described above with respect to the kernels that produce its segment. */
#define VETR_SEG_DESC 1
#define VETR_SEG_POINTS 2
#define VETR_SEG_CONF 4
int vetr_exchange_finalize_part(vetr_ctx* ctx, const vetr_exchange* ex, int channels, int n_tex, int n, int segments,
                                int ctas_per_sm);

/* Error-grid rasterisation: PointRendererCache::FillSceneGridWithLoss -> FillSceneGridWithLossRasterize
 * (RenderForward.cu:639-791; called per image from train.cpp:1077 before the tomography's point spawning).  For every
 * cell of the scene grid whose eight box corners lie in front of the camera of `view`, the pixels of its projected box
 * (the twelve triangles of its faces, inside the image minus a 32-pixel border) add sum_c |loss_img[c,y,x]| to
 * cell_value and 1 to cell_access_count.  Both arrays are accumulated into (the caller zeroes them per epoch and
 * divides afterwards, NeuralPointCloudCuda.h:42-52).
 *   cell_bb_min, cell_bb_len [n_cells,3] float (t_cell_bb_min, t_cell_bb_length); loss_img [channels, view->h, view->w]
 *   cell_value [n_cells] float; cell_access_count [n_cells] int32.
 * Counts are exact; values are float sums in no fixed order (as in the reference). */
int vetr_grid_loss(vetr_ctx* ctx, const vetr_cameras* cameras, const vetr_view* view, float dist_cutoff, int n_cells,
                   const float* cell_bb_min, const float* cell_bb_len, const float* loss_img, int channels,
                   float* cell_value, int32_t* cell_access_count);

/* Texture environment map: EnvironmentMapImpl::Sample2 (rendering/EnvironmentMap.cu:378-485) with its kernels
 * BuildSphericalRayList (:201-287, pinhole branch) and CreateSampleUVMapAllSpheres (:587-684) and the libtorch operators
 * of forward_mps5 (:692-758: two 3-D grid_sample calls, sigmoid, one multiply-add chain per sphere), as ONE kernel over
 * all views, levels and pixels; the backward call replaces what autograd records for forward_mps5.
 * The map is n_spheres concentric spheres around the origin (the last one at infinity), each an equirectangular
 * resolution x resolution texture of a density and `channels` colours.  For a pixel of level l, the ray through it is
 * intersected with every sphere from the inside, the hit direction gives (u, v) = (lon / pi, 2 lat / pi), the sphere gives
 * z = 2 s / (n_spheres - 1) - 1, and the textures are sampled at (u, v, z) exactly as
 * grid_sample(mode = bilinear, padding_mode = zeros, align_corners = true) does on the 5-D parameters.  Front to back,
 *     env[c] += T * alpha_s * color_s[c];  T *= 1 - alpha_s;   alpha_s = hit_s * sigmoid(density_s), 1 on the last sphere,
 * starting from T = the rasterizer's final transmittance of the pixel (LayerCuda::weight, RenderModule.cpp:130-141).
 * A sphere the ray misses (possible only from outside it) contributes nothing; the reference's value there is NaN. */
typedef struct vetr_envmap
{
    const float* density;  /* [n_spheres, resolution, resolution]            (EnvironmentMapImpl::density, [1,1,S,R,R]) */
    const float* color;    /* [channels, n_spheres, resolution, resolution]  (EnvironmentMapImpl::color, [1,C,S,R,R]) */
    float        radii[8]; /* inner_radius * radius_factor^s (EnvironmentMap.cu:109-113); the last sphere's is unused */
    int32_t      n_spheres, resolution, channels; /* n_spheres 1..8 (MAX_NUM_SPHERES), channels 1..4 */
    int32_t      up_axis;             /* 0, 1 or 2: the axis the latitude is measured from (EnvironmentMap.cu:543-563) */
    int32_t      non_subzero_texture; /* 1: |color| is sampled (EnvironmentMap.cu:728) */
} vetr_envmap;
#define VETR_ENV_ADD 1            /* out += env instead of out = env: `images[i] + env_maps[i]`, RenderModule.cpp:188-203 */
#define VETR_ENV_NOT_AT_POINTS 2  /* no_envmap_at_points: env counts as 0 where weight > 0.001 (RenderModule.cpp:190-201) */
#define VETR_ENV_DEPTH_TEST_WEIGHT 4 /* mode 0 (FUZZY_DT), where weight is a hit count: T starts at (weight > 0.5 ? 0 : 1);
                                        with VETR_ENV_ADD, out is also zeroed where weight <= 0.5 (RenderModule.cpp:143-155) */
#define VETR_ENV_NO_DISTORTION_CHECK 8 /* the caller vouches that the views' cameras have zero distortion coefficients: the
                                          call then does not read the intrinsics back (no synchronisation; capturable) */
/*   weight   num_layers device pointers [n_views,1,h_l,w_l] (out_weight of vetr_forward)
 *   out      num_layers device pointers [n_views,channels,h_l,w_l]
 * All views share views[0].w x views[0].h; level sizes halve with integer division (EnvironmentMap.cu:398-436).
 * Pinhole cameras only; non-zero distortion coefficients return VETR_E_UNSUPPORTED (the reference inverts the
 * distortion with an iteration whose source is not part of its tree); checking that copies the intrinsics to the host
 * and synchronises the stream unless VETR_ENV_NO_DISTORTION_CHECK is given. */
int vetr_envmap_forward(vetr_ctx* ctx, const vetr_cameras* cameras, const vetr_view* views, int n_views, int num_layers,
                        const vetr_envmap* env, const float* const* weight, float* const* out, int flags);
/* Gradients of the map's parameters for the incoming gradient of `out` (same shapes), ADDED to
 *   g_density [n_spheres, resolution, resolution],  g_color [channels, n_spheres, resolution, resolution].
 * Nothing else receives a gradient in the reference either: the rays come from a raw kernel and the transmittance is a
 * detached copy (RenderModule.cpp:140).  flags as in the forward call (VETR_ENV_ADD is ignored).  fp32 sums in no fixed
 * order; lanes of a warp that hit the same texel are summed before the one atomic per texel and value. */
int vetr_envmap_backward(vetr_ctx* ctx, const vetr_cameras* cameras, const vetr_view* views, int n_views, int num_layers,
                         const vetr_envmap* env, const float* const* weight, const float* const* grad_out, int flags,
                         float* g_density, float* g_color);

/* Drop-out radius of every point: SceneData::ComputeRadius (data/SceneData.cpp:554-597), which the reference runs on the
 * host (a KD-tree over the whole cloud, one (k+1)-nearest query per point) when a scene is prepared and again whenever
 * points are added (NeuralScene.cpp:511, 1079; SceneData.cpp:756, 812).  radius[i] = |p_i - p_j| for the k-th nearest other point j, i.e. the
 * (k+1)-th smallest distance from p_i to the points of the cloud, itself included; with fewer than k+1 points, the distance
 * to the farthest one.  The value does not depend on how equal distances are ordered, and the squared distance is formed
 * as (dx dx + dy dy) + dz dz in fp32 without contraction, so results are bit-equal to an all-pairs evaluation.
 *   position  n points, `position_stride` floats apart (4 for t_position [N,4]); finite coordinates
 *   radius    written at radius[i * radius_stride] (position + 3 with stride 4 writes t_position's radius column in place)
 *   k         1..16 (the reference uses 4)
 * The call bins the points into a uniform grid whose cell size it picks from the cloud (a few host round trips of a few
 * bytes each), so it synchronises the context's stream; its scratch (24 bytes per point and 8 bytes per grid cell, at
 * most 64 Mi cells) is allocated inside the context and reused by later calls. */
int vetr_knn_radius(vetr_ctx* ctx, const float* position, int position_stride, int n, int k, float* radius, int radius_stride);

/* Removing points: NeuralScene::RemovePoints (data/NeuralScene.cpp:1156-1239) without the host round trip.  The reference
 * sorts the indices to remove, forms the complementary keep list in a host loop, rebuilds the cloud through a CPU mesh and
 * index_selects every per-point tensor with the keep list (texture and confidence, NeuralTexture.cpp:160-173; the Adam
 * moments, my_adam.cpp:107-135).  Here the plan call flags the removed points and scans the flags, and one gather call per
 * group of tensors copies the survivors in their old order: dst[r, new_index[i], :] = src[r, i, :].
 *   remove     m device int64 indices (the reference's index dtype), duplicates allowed; an index outside [0, n) returns
 *              VETR_E_INVALID_ARG
 *   new_index  [n] device int32, written: the index of point i after the removal, or -1
 *   n_kept     host int, written (the call synchronises the stream to read it): the caller sizes the destinations with it */
int vetr_remove_points_plan(vetr_ctx* ctx, int n, const int64_t* remove, int m, int32_t* new_index, int* n_kept);
typedef struct vetr_point_array
{
    const void* src; /* [rows, n, width] elements of four bytes (float or int32) */
    void*       dst; /* [rows, n_kept, width]; must not overlap src */
    int32_t     rows, width; /* t_position [N,4]: rows 1, width 4 (16-byte aligned); texture [C,N]: rows C, width 1 */
} vetr_point_array;
int vetr_gather_points(vetr_ctx* ctx, int n, int n_kept, const int32_t* new_index, const vetr_point_array* arrays, int n_arrays);

/* L1 loss of an output pyramid against a target pyramid and its gradient, one launch for all levels:
 *   loss = sum_l mean |image_l - target_l| (written to the device scalar `loss`), grad_l = sign(image_l - target_l) / numel_l.
 * No counterpart in the reference's rasterizer: its training loop forms this term with libtorch element-wise operators
 * between PointRender's forward and backward; the benchmark's step does the same with this call.
 * image, target, grad: num_levels device pointers (16-byte aligned) of numel[l] floats each. */
int vetr_l1_loss_grad(vetr_ctx* ctx, int num_levels, const float* const* image, const float* const* target,
                      float* const* grad, const int64_t* numel, float* loss);

/* ApplyTangentToPose (PointRenderer.cu:1325-1349): poses[i] <- exp_se3(tangent[i]) * poses[i]; tangent[i] <- 0. */
int vetr_apply_tangent(vetr_ctx* ctx, double* tangent /*[n,6]*/, double* poses_se3 /*[n,8]*/, int n);

/* Copies the device status words of `lists` to the host (synchronises the stream).  Returns VETR_E_LIST_OVERFLOW
 * if the last forward call produced more fragments than lists->capacity. */
int vetr_read_status(vetr_ctx* ctx, const vetr_lists* lists, int64_t* total_fragments, int32_t* longest_list);

/* Parity / debugging: unpacks one (view, level) of `lists` into the reference's collections layout [2,F_l] int32
 * (row 0 depth bits, row 1 point index; PointRenderer.cu:817-818) and its scanned_counting [h_l*w_l].
 * Synchronises.  out_collections may be NULL to query *n_fragments only. */
int vetr_get_lists(vetr_ctx* ctx, const vetr_lists* lists, int w, int h, int num_layers, int n_views, int view,
                   int layer, int32_t* out_collections, int32_t* out_scanned_counting, int64_t* n_fragments);

/* The scan of the forward pass (per-pixel counts -> list offsets, total fragment count, longest list, work-item table)
 * as a call of its own that allocates nothing.  It has no counterpart in the reference; it exists for hosts that cannot
 * allocate device memory while they render (a frame loop that cannot take the device-wide stall of cudaMalloc, a process
 * whose device memory was handed out once by an arena, a region where allocation is forbidden).  The scan's scratch, one
 * partial sum per 4096 pixels, is a fixed 128 KB array inside the library image on every GPU that loads it.
 *   limit       n_pixels <= 67 108 864 (16384 tiles); more returns VETR_E_TOO_LARGE
 *   inputs      counts [n_pixels] int32 device array; capacity as in vetr_lists
 *   outputs     ends [n_pixels] = exclusive scan of counts (the start of every list; vetr_forward's collection pass later
 *               advances its copy to the list ends); status [4] = {total, overflow flag, longest list, work items};
 *               items [items_capacity >= vetr_item_table_entries(capacity, n_pixels)]
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and should therefore come before
 * any stream capture on that device; it is not safe to make that first call from two threads at once.  The kernels are
 * launched on `device`; the caller's current device is the same after the call as before it.  All calls share
 * the one array: it is fully rewritten by every call (nothing needs clearing), the status words are zeroed by the call,
 * and two calls whose kernels overlap on the GPU (different streams, same device) race.  Calls no cudaMalloc / cudaFree. */
int vetr_scan_counts_static(int device, void* cuda_stream, const int32_t* counts, int64_t n_pixels, int64_t capacity,
                            int32_t* ends, int32_t* status, int32_t* items, int64_t items_capacity);

/* Measurement hooks (the reference wraps every pass in a CudaTimerSystem scope, e.g. PointRenderer.cu:770,843,872,886).
 * With timing enabled every kernel of vetr_forward / vetr_backward / vetr_finalize_gradients is bracketed by CUDA events
 * on the context's stream.  vetr_get_timings() synchronises and returns the milliseconds of the most recent launch of each
 * kernel, indexed by VETR_T_*; entries that did not run are 0. */
enum
{
    VETR_T_COUNT = 0,    /* project + count */
    VETR_T_SCAN,         /* the three scan kernels */
    VETR_T_COLLECT,      /* project + collect */
    VETR_T_SORT_BLEND,   /* sort + blend */
    VETR_T_BACKWARD,     /* backward */
    VETR_T_FINALIZE,     /* transpose + normalisation kernels */
    VETR_T_POINT_BACKWARD, /* per-point pass of the backward step (modes 1 and 2) */
    VETR_T_EXCHANGE,     /* vetr_exchange_finalize */
    VETR_T_ENVMAP,       /* vetr_envmap_forward / vetr_envmap_backward */
    VETR_T_KNN,          /* vetr_knn_radius */
    VETR_T_N
};
int vetr_set_timing(vetr_ctx* ctx, int enable);
int vetr_get_timings(vetr_ctx* ctx, float* out_ms /*[VETR_T_N]*/);

/* Number of kernels this context has launched since it was created. */
int64_t vetr_launch_count(const vetr_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* VETR_H */
