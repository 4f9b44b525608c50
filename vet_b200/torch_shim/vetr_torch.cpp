// See vetr_torch.h.  Sequencing follows BlendPointCloudForward / BlendPointCloudBackward
// (rendering/PointRenderer.cu:657-1069, 1111-1323); all arithmetic happens behind the C ABI.
#include "vetr_torch.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace vetr_torch
{
namespace
{
void check(int status, const char* where)
{
    if (status != VETR_OK) throw std::runtime_error(std::string(where) + ": " + vetr_strerror(status));
}

vetr_params make_params(const NeuralRenderInfo& info)
{
    const RenderParams& p = info.params;
    if (p.check_normal) throw std::runtime_error("vetr: check_normal is not supported");
    vetr_params q{};
    q.render_mode                  = p.render_mode;
    q.num_layers                   = info.num_layers;
    q.num_channels                 = p.num_texture_channels;
    q.drop_out_points_by_radius    = p.drop_out_points_by_radius;
    q.drop_out_radius_threshold    = p.drop_out_radius_threshold;
    q.dist_cutoff                  = p.dist_cutoff;
    q.use_environment_map          = p.use_environment_map;
    q.viewer_only                  = p.viewer_only;
    q.stability_cutoff_value       = p.stability_cutoff_value;
    q.debug_max_list_length        = p.debug_max_list_length;
    q.need_point_gradient          = p.need_point_gradient;
    q.K_gradient_factor            = p.K_gradient_factor;
    q.distortion_gradient_factor   = p.distortion_gradient_factor;
    q.output_background_mask_value = p.output_background_mask_value;
    q.background_alpha_to_point0   = 1;
    q.keep_sorted_lists            = 1;
    q.depth_accept_blend           = p.depth_accept_blend;
    q.depth_accept                 = p.depth_accept;
    q.ghost_gradients              = p.ghost_gradients;
    return q;
}

std::vector<vetr_view> make_views(const NeuralRenderInfo& info, int b0, int b1)
{
    std::vector<vetr_view> v;
    for (int b = b0; b < b1; ++b)
    {
        const ReducedImageInfo& im = info.images[b];
        vetr_view x{};
        x.w = im.w, x.h = im.h, x.image_index = im.image_index, x.camera_index = im.camera_index;
        x.camera_model = im.camera_model_type;
        for (int i = 0; i < 5; ++i) x.crop[i] = im.crop_transform[i];
        for (int i = 0; i < 4; ++i) x.rot[i] = im.crop_rotation[i];
        v.push_back(x);
    }
    return v;
}

struct Inputs
{
    vetr_cloud cloud;
    vetr_texture tex;
    vetr_cameras cams;
    torch::Tensor index, confidence;  // contiguous views kept alive
};

Inputs make_inputs(const RenderScene& s)
{
    TORCH_CHECK(s.t_position.is_cuda() && s.t_position.is_contiguous() && s.t_position.dtype() == torch::kFloat32);
    TORCH_CHECK(s.texture.is_contiguous() && s.poses_se3.dtype() == torch::kFloat64 && s.poses_se3.is_contiguous());
    Inputs in;
    in.index      = s.t_index.reshape({-1}).contiguous();
    in.confidence = s.confidence_value_of_point.reshape({-1}).contiguous();
    in.cloud      = {s.t_position.data_ptr<float>(), in.index.data_ptr<int>(), (int)s.t_position.size(0)};
    in.tex        = {s.texture.data_ptr<float>(), in.confidence.data_ptr<float>(), s.background_color.data_ptr<float>(),
                     (int)s.texture.size(1)};
    in.cams       = {s.poses_se3.data_ptr<double>(), s.intrinsics.data_ptr<float>(), (int)s.poses_se3.size(0),
                     (int)s.intrinsics.size(0)};
    return in;
}

struct GroupLists
{
    torch::Tensor counts, ends, frags, status, items, level_mask;
    vetr_lists c;
};

GroupLists alloc_lists(int64_t n_pixels, int64_t capacity, int64_t mask_entries, const torch::Device& dev)
{
    auto i32 = torch::TensorOptions().device(dev).dtype(torch::kInt32);
    GroupLists g;
    g.counts = torch::empty({n_pixels}, i32);
    g.ends   = torch::empty({n_pixels}, i32);
    g.frags  = torch::empty({std::max<int64_t>(capacity, 1), 4}, i32.dtype(torch::kInt64));
    g.status = torch::zeros({4}, i32);
    int64_t n_items = vetr_item_table_entries(capacity, n_pixels);
    g.items  = torch::empty({n_items}, i32);
    g.level_mask = torch::empty({std::max<int64_t>(mask_entries, 1)}, i32.dtype(torch::kUInt8));
    g.c = {g.counts.data_ptr<int>(), g.ends.data_ptr<int>(), g.frags.data_ptr(), capacity, g.status.data_ptr<int>(),
           g.items.data_ptr<int>(), n_items, mask_entries > 0 ? g.level_mask.data_ptr<uint8_t>() : nullptr, nullptr, nullptr};
    return g;
}

std::vector<float*> level_ptrs(const std::vector<torch::Tensor>& t, int b0)
{
    std::vector<float*> p;
    for (auto& x : t) p.push_back(x.data_ptr<float>() + (int64_t)b0 * x.stride(0));
    return p;
}
}  // namespace

PointRendererCache::~PointRendererCache()
{
    if (ctx_) vetr_destroy(ctx_);
    if (status_host_)
    {
        cudaFreeHost(status_host_);
        for (auto& e : status_event_) cudaEventDestroy(e);
    }
}

vetr_ctx* PointRendererCache::context(int device)
{
    void* stream = (void*)at::cuda::getCurrentCUDAStream(device).stream();
    if (!ctx_ || device_ != device)
    {
        if (ctx_) vetr_destroy(ctx_);
        check(vetr_create(&ctx_, device, stream), "vetr_create");
        device_ = device;
    }
    check(vetr_set_stream(ctx_, stream), "vetr_set_stream");
    return ctx_;
}

int64_t PointRendererCache::FragmentCapacity(int64_t safe_bound, int n_views, int n_points, int num_layers, int w, int h, int mode)
{
    const int64_t shape[5] = {n_points, num_layers, w, h, mode};
    if (!std::equal(shape, shape + 5, shape_))  // another cloud, pyramid or mode: what was seen says nothing about it
    {
        std::copy(shape, shape + 5, shape_);
        high_water_per_view_ = 0;
    }
    int64_t cap = safe_bound;
    if (high_water_per_view_ > 0 && mode != VETR_MODE_FUZZY_DT)  // (mode 0 keeps one record per pixel, not lists)
        cap = std::min<int64_t>(safe_bound, (int64_t)(kFragmentHeadroom * (double)high_water_per_view_ * n_views) + 4096);
    last_fragment_capacity = cap;
    return cap;
}

void PointRendererCache::NoteStatus(const torch::Tensor& status_dev, int64_t capacity, int n_views, bool after_backward)
{
    if (pending_.size() >= kStatusSlots) CheckEarlierCalls();
    if (!status_host_)
    {
        // plain runtime objects, not tensors: a cache may live in static storage and be destroyed after libtorch's own
        // allocators, and the runtime's calls fail harmlessly then
        TORCH_CHECK(cudaMallocHost((void**)&status_host_, kStatusSlots * 4 * sizeof(int)) == cudaSuccess, "vetr: no pinned memory");
        for (auto& e : status_event_) TORCH_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess);
    }
    const int slot = (int)pending_.size();
    cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
    TORCH_CHECK(cudaMemcpyAsync(status_host_ + 4 * slot, status_dev.data_ptr<int>(), 4 * sizeof(int), cudaMemcpyDeviceToHost, st) ==
                cudaSuccess);
    TORCH_CHECK(cudaEventRecord(status_event_[slot], st) == cudaSuccess);
    pending_.push_back({slot, capacity, n_views, after_backward});
}

void PointRendererCache::CheckEarlierCalls()
{
    std::string problem;
    for (auto& p : pending_)
    {
        cudaEventSynchronize(status_event_[p.slot]);  // recorded one call ago: already complete
        const int* w = status_host_ + 4 * p.slot;
        if (!p.after_backward && render_mode != FUZZY_DT)
            high_water_per_view_ = std::max<int64_t>(high_water_per_view_, ((int64_t)w[0] + p.n_views - 1) / std::max(p.n_views, 1));
        if (w[1] & 1)
        {
            high_water_per_view_ = 0;  // the next call is sized by the bound that cannot overflow
            problem = "vetr: the fragment buffer of the previous render call overflowed (" + std::to_string(w[0]) + " fragments, room for " +
                      std::to_string(p.capacity) + "); its images are incomplete.  The next call is sized safely: run the step again";
        }
        else if ((w[1] & 2) && p.after_backward)
            problem = "vetr: the mode-2 backward pass skipped at least one list of more than 4096 fragments (longest list " +
                      std::to_string(w[2]) + "); its gradients are incomplete";
    }
    pending_.clear();
    if (!problem.empty()) throw std::runtime_error(problem);
}

void PointRendererCache::FillSceneGridWithLoss(int batch, RenderScene& s, const std::vector<ReducedImageInfo>& images,
                                               torch::Tensor loss_img, float dist_cutoff)
{
    TORCH_CHECK(batch >= 0 && batch < (int)images.size(), "FillSceneGridWithLoss: batch index out of range");
    TORCH_CHECK(s.t_cell_bb_min.defined() && s.t_cell_bb_length.defined() && s.t_cell_value.defined() &&
                    s.t_cell_access_count.defined(),
                "FillSceneGridWithLoss: the scene has no grid");
    TORCH_CHECK(loss_img.dim() == 3 && loss_img.dtype() == torch::kFloat32, "loss image must be [C,h,w] float");
    TORCH_CHECK(s.t_cell_value.dtype() == torch::kFloat32 && s.t_cell_access_count.dtype() == torch::kInt32);
    TORCH_CHECK(s.t_cell_value.is_contiguous() && s.t_cell_access_count.is_contiguous(), "grid tensors must be contiguous");
    const auto dev = s.t_cell_bb_min.device();
    c10::cuda::CUDAGuard guard(dev);
    vetr_ctx* vc = context(dev.index());
    const ReducedImageInfo& im = images[batch];
    TORCH_CHECK(loss_img.size(1) == im.h && loss_img.size(2) == im.w, "loss image does not match the view");
    vetr_view v{};
    v.w = im.w, v.h = im.h, v.image_index = im.image_index, v.camera_index = im.camera_index;
    v.camera_model = im.camera_model_type;
    for (int i = 0; i < 5; ++i) v.crop[i] = im.crop_transform[i];
    for (int i = 0; i < 4; ++i) v.rot[i] = im.crop_rotation[i];
    torch::Tensor bb_min = s.t_cell_bb_min.contiguous(), bb_len = s.t_cell_bb_length.contiguous(), loss = loss_img.contiguous();
    torch::Tensor poses = s.poses_se3.contiguous(), intr = s.intrinsics.contiguous();
    vetr_cameras cams{poses.data_ptr<double>(), intr.data_ptr<float>(), (int)poses.size(0), (int)intr.size(0)};
    check(vetr_grid_loss(vc, &cams, &v, dist_cutoff, (int)bb_min.size(0), bb_min.data_ptr<float>(), bb_len.data_ptr<float>(),
                         loss.data_ptr<float>(), (int)loss.size(0), s.t_cell_value.data_ptr<float>(),
                         s.t_cell_access_count.data_ptr<int>()),
          "vetr_grid_loss");
}

std::vector<torch::Tensor> BlendPointCloud(NeuralRenderInfo* info)
{
    torch::intrusive_ptr<NeuralRenderInfo> render_data = torch::make_intrusive<NeuralRenderInfo>(*info);
    TORCH_CHECK(render_data->scene, "BlendPointCloud: no scene");
    RenderScene& s = *render_data->scene;
    return torch::autograd::PointRender::apply(s.texture, s.background_color, s.t_position, s.tangent_poses, s.intrinsics,
                                               s.confidence_value_of_point, s.dynamic_refinement_t,
                                               torch::IValue(render_data));
}

void ApplyTangentToPose(torch::Tensor tangent, torch::Tensor pose)
{
    TORCH_CHECK(tangent.is_contiguous() && pose.is_contiguous() && tangent.dtype() == torch::kFloat64);
    c10::cuda::CUDAGuard guard(pose.device());
    vetr_ctx* ctx = nullptr;
    check(vetr_create(&ctx, pose.device().index(), (void*)at::cuda::getCurrentCUDAStream().stream()), "vetr_create");
    int rc = vetr_apply_tangent(ctx, tangent.data_ptr<double>(), pose.data_ptr<double>(), (int)tangent.size(0));
    vetr_destroy(ctx);
    check(rc, "vetr_apply_tangent");
}
}  // namespace vetr_torch

namespace torch::autograd
{
using namespace vetr_torch;

variable_list PointRender::forward(AutogradContext* ctx, Variable texture, Variable background_color, Variable points,
                                   Variable pose_tangents, Variable intrinsics, Variable confidence,
                                   Variable dynamic_refinement, IValue info_v)
{
    ctx->saved_data["render_info"] = info_v;
    NeuralRenderInfo* info = info_v.toCustomClass<NeuralRenderInfo>().get();
    TORCH_CHECK(info->cache, "NeuralRenderInfo::cache is not set");
    PointRendererCache& cache = *info->cache;
    RenderScene& s            = *info->scene;
    const auto dev            = s.t_position.device();
    c10::cuda::CUDAGuard guard(dev);
    vetr_ctx* vc = cache.context(dev.index());

    const int B = (int)info->images.size(), L = info->num_layers, C = info->params.num_texture_channels;
    TORCH_CHECK(B > 0);
    cache.CheckEarlierCalls();
    cache.num_batches = B;
    cache.render_mode = (PointRendererCache::RenderMode)info->params.render_mode;
    const vetr_params prm = make_params(*info);
    Inputs in             = make_inputs(s);

    auto f32 = torch::TensorOptions().device(dev).dtype(torch::kFloat32);
    std::vector<torch::Tensor> color, weight, depth, mask;
    cache.layers_cuda.resize(L);
    int w = info->images.front().w, h = info->images.front().h;
    for (int l = 0; l < L; ++l, w /= 2, h /= 2)
    {
        TORCH_CHECK(w > 0 && h > 0, "pyramid level of size 0");
        color.push_back(torch::empty({B, C, h, w}, f32));
        weight.push_back(torch::empty({B, 1, h, w}, f32));
        depth.push_back(torch::empty({B, 1, h, w}, f32));
        if (info->params.output_background_mask) mask.push_back(torch::empty({B, 1, h, w}, f32));
        cache.layers_cuda[l].w = w, cache.layers_cuda[l].h = h;
        cache.layers_cuda[l].weight = weight.back(), cache.layers_cuda[l].depth = depth.back();
    }

    // drop-out mask like PointRendererCache::InitializeData (PointRenderer.cu:461-468)
    torch::Tensor dropout;
    if (info->params.dropout > 0 && info->train)
    {
        dropout = torch::empty({B, s.t_position.size(0)}, f32).bernoulli_(info->params.dropout);
        cache.dropout_points = dropout;
    }

    const int64_t P = vetr_pyramid_pixels(info->images.front().w, info->images.front().h, L);
    std::vector<torch::Tensor> saved = {texture, background_color, points, intrinsics, confidence};
    for (auto& c : color) saved.push_back(c);
    int n_groups = 0;
    for (int b0 = 0; b0 < B; b0 += VETR_MAX_VIEWS, ++n_groups)
    {
        const int b1 = std::min(B, b0 + VETR_MAX_VIEWS), nb = b1 - b0;
        const bool point_pass = prm.render_mode == VETR_MODE_BILINEAR_BLEND ||
                                ((prm.render_mode == VETR_MODE_FULL_BLEND || prm.render_mode == VETR_MODE_FUZZY_BLEND) &&
                                 prm.need_point_gradient);
        const int w0 = info->images.front().w, h0 = info->images.front().h;
        const int64_t capacity = cache.FragmentCapacity(vetr_list_capacity(in.cloud.n, nb, w0, h0, &prm), nb, in.cloud.n, L, w0, h0,
                                                        prm.render_mode);
        GroupLists g = alloc_lists(P * nb, capacity, point_pass ? (int64_t)nb * in.cloud.n : 0, dev);
        auto views   = make_views(*info, b0, b1);
        auto pc = level_ptrs(color, b0), pw = level_ptrs(weight, b0), pd = level_ptrs(depth, b0), pm = level_ptrs(mask, b0);
        check(vetr_forward(vc, &prm, &in.cloud, &in.tex, &in.cams, views.data(), nb,
                           dropout.defined() ? dropout.data_ptr<float>() + (int64_t)b0 * dropout.stride(0) : nullptr, &g.c,
                           pc.data(), pw.data(), mask.empty() ? nullptr : pm.data(), pd.data()),
              "vetr_forward");
        cache.NoteStatus(g.status, capacity, nb, false);
        for (auto& t : {g.counts, g.ends, g.frags, g.status, g.items, g.level_mask}) saved.push_back(t);
    }
    // the drop-out mask belongs to this call (PointRenderer.cu:1056, 1194 save it with the node): a second forward through
    // the same cache before this call's backward must not replace it
    saved.push_back(dropout.defined() ? dropout : torch::empty({0}, f32));
    ctx->saved_data["n_groups"] = n_groups;
    ctx->save_for_backward(saved);

    variable_list out = color;
    if (info->params.add_depth_to_network) out.insert(out.end(), depth.begin(), depth.end());
    out.insert(out.end(), mask.begin(), mask.end());
    return out;
}

variable_list PointRender::backward(AutogradContext* ctx, variable_list grad_output)
{
    IValue info_v          = ctx->saved_data["render_info"];
    NeuralRenderInfo* info = info_v.toCustomClass<NeuralRenderInfo>().get();
    PointRendererCache& cache = *info->cache;
    RenderScene& s            = *info->scene;
    const auto dev            = s.t_position.device();
    c10::cuda::CUDAGuard guard(dev);
    vetr_ctx* vc = cache.context(dev.index());
    const int B = (int)info->images.size(), L = info->num_layers, C = info->params.num_texture_channels;
    const vetr_params prm = make_params(*info);
    Inputs in             = make_inputs(s);
    auto saved            = ctx->get_saved_variables();
    const int n_groups    = (int)ctx->saved_data["n_groups"].toInt();
    TORCH_CHECK((int)saved.size() == 5 + L + 6 * n_groups + 1);
    cache.CheckEarlierCalls();  // an overflow of this call's forward pass is reported before gradients are formed from it
    const torch::Tensor dropout = saved.back();

    std::vector<torch::Tensor> color(saved.begin() + 5, saved.begin() + 5 + L), gcolor;
    for (int l = 0; l < L; ++l)
    {
        TORCH_CHECK(grad_output[l].defined() && grad_output[l].dtype() == torch::kFloat32);
        gcolor.push_back(grad_output[l].contiguous());
    }
    const int64_t n = s.t_position.size(0), n_tex = s.texture.size(1);
    auto f32 = torch::TensorOptions().device(dev).dtype(torch::kFloat32);
    // accumulation buffers (point-major) and the reference's output tensors
    torch::Tensor g_desc = torch::zeros({n_tex, 4}, f32), g_conf = torch::zeros({1, n_tex}, f32);
    torch::Tensor g_background = torch::zeros_like(s.background_color);
    torch::Tensor g_points, g_pose, g_pose_count, g_intr, g_intr_count;
    if (s.t_position.requires_grad()) g_points = torch::zeros({n, 4}, f32);
    if (s.tangent_poses.requires_grad())
    {
        g_pose       = torch::zeros_like(s.tangent_poses);
        g_pose_count = torch::zeros({s.tangent_poses.size(0)}, f32);
    }
    if (s.intrinsics.requires_grad())
    {
        g_intr       = torch::zeros_like(s.intrinsics);
        g_intr_count = torch::zeros({s.intrinsics.size(0)}, f32);
    }
    for (int gi = 0, b0 = 0; gi < n_groups; ++gi, b0 += VETR_MAX_VIEWS)
    {
        const int b1 = std::min(B, b0 + VETR_MAX_VIEWS), nb = b1 - b0;
        auto* t = &saved[5 + L + 6 * gi];
        // scratch of the per-point pass that forms the position / pose / intrinsics gradients of modes 1 and 2
        torch::Tensor point_grad;
        if (prm.render_mode == VETR_MODE_BILINEAR_BLEND)
            point_grad = torch::empty({(int64_t)nb * L * n * 4}, f32);  // one value per bilinear corner
        else if ((prm.render_mode == VETR_MODE_FULL_BLEND || prm.render_mode == VETR_MODE_FUZZY_BLEND) && prm.need_point_gradient)
            point_grad = torch::empty({(int64_t)nb * L * n * 2}, f32);
        torch::Tensor pixel_scratch = torch::empty({std::max<int64_t>(t[0].size(0), 1) * 8}, f32);
        vetr_lists lists = {t[0].data_ptr<int>(), t[1].data_ptr<int>(), t[2].data_ptr(), t[2].size(0), t[3].data_ptr<int>(),
                            t[4].data_ptr<int>(), t[4].size(0), t[5].data_ptr<uint8_t>(),
                            point_grad.defined() ? point_grad.data_ptr<float>() : nullptr, pixel_scratch.data_ptr<float>()};
        auto views = make_views(*info, b0, b1);
        auto pc = level_ptrs(color, b0), pg = level_ptrs(gcolor, b0);
        std::vector<const float*> cpc(pc.begin(), pc.end()), cpg(pg.begin(), pg.end());
        const bool has_dropout = dropout.numel() > 0;
        check(vetr_backward(vc, &prm, &in.cloud, &in.tex, &in.cams, views.data(), nb,
                            has_dropout ? dropout.data_ptr<float>() + (int64_t)b0 * dropout.stride(0) : nullptr,
                            &lists, cpc.data(), cpg.data(),
                            g_desc.data_ptr<float>(), g_conf.data_ptr<float>(),
                            g_points.defined() ? g_points.data_ptr<float>() : nullptr, g_background.data_ptr<float>(),
                            g_pose.defined() ? g_pose.data_ptr<double>() : nullptr,
                            g_pose.defined() ? g_pose_count.data_ptr<float>() : nullptr,
                            g_intr.defined() ? g_intr.data_ptr<float>() : nullptr,
                            g_intr.defined() ? g_intr_count.data_ptr<float>() : nullptr),
              "vetr_backward");
        // mode 2 flags lists it had to skip in the status words: looked at when the next call starts
        if (prm.render_mode == VETR_MODE_FUZZY_BLEND) cache.NoteStatus(t[3], t[2].size(0), nb, true);
    }
    torch::Tensor g_texture = torch::empty_like(s.texture);
    check(vetr_finalize_gradients(vc, C, (int)n_tex, g_desc.data_ptr<float>(), g_texture.data_ptr<float>(), (int)n,
                                  g_points.defined() ? g_points.data_ptr<float>() : nullptr, nullptr,
                                  g_pose.defined() ? (int)g_pose.size(0) : 0,
                                  g_pose.defined() ? g_pose.data_ptr<double>() : nullptr,
                                  g_pose.defined() ? g_pose_count.data_ptr<float>() : nullptr,
                                  g_intr.defined() ? (int)g_intr.size(0) : 0,
                                  g_intr.defined() ? g_intr.data_ptr<float>() : nullptr,
                                  g_intr.defined() ? g_intr_count.data_ptr<float>() : nullptr),
          "vetr_finalize_gradients");
    // order of BlendPointCloudBackward's return (PointRenderer.cu:1319-1322) + one empty gradient for the IValue
    return {g_texture, g_background, g_points, g_pose, g_intr, g_conf.view_as(s.confidence_value_of_point), Variable(), Variable()};
}
}  // namespace torch::autograd

// ---------------------------------------------------------------------------------------------------------
// Drop-out radius

namespace vetr_torch
{
torch::Tensor ComputeRadius(torch::Tensor position, int n)
{
    TORCH_CHECK(position.is_cuda() && position.dtype() == torch::kFloat32 && position.dim() == 2 &&
                    (position.size(1) == 3 || position.size(1) == 4),
                "ComputeRadius: position must be a CUDA float tensor [N,3] or [N,4]");
    static PointRendererCache cache;  // owns the context and its grid scratch
    c10::cuda::CUDAGuard guard(position.device());
    vetr_ctx* vc = cache.context(position.device().index());
    torch::Tensor p = position.contiguous();
    torch::Tensor r = torch::empty({p.size(0)}, p.options());
    check(vetr_knn_radius(vc, p.data_ptr<float>(), (int)p.size(1), (int)p.size(0), n, r.data_ptr<float>(), 1), "vetr_knn_radius");
    return r;
}
}  // namespace vetr_torch

// ---------------------------------------------------------------------------------------------------------
// Point removal

namespace vetr_torch
{
int64_t RemovePoints(RenderScene& s, torch::Tensor indices_to_remove, std::vector<torch::Tensor> per_point_state)
{
    TORCH_CHECK(s.t_position.defined() && s.t_position.is_cuda() && s.t_position.dim() == 2 && s.t_position.size(1) == 4,
                "RemovePoints: t_position must be a CUDA tensor [N,4]");
    static PointRendererCache cache;
    const auto dev = s.t_position.device();
    c10::cuda::CUDAGuard guard(dev);
    vetr_ctx* vc = cache.context(dev.index());
    torch::NoGradGuard ngg;
    const int n = (int)s.t_position.size(0);
    torch::Tensor remove = indices_to_remove.to(dev, torch::kLong).reshape({-1}).contiguous();
    torch::Tensor new_index = torch::empty({std::max(n, 1)}, torch::TensorOptions().dtype(torch::kInt32).device(dev));
    int kept = 0;
    check(vetr_remove_points_plan(vc, n, remove.numel() ? remove.data_ptr<int64_t>() : nullptr, (int)remove.numel(),
                                  new_index.data_ptr<int>(), &kept),
          "vetr_remove_points_plan");
    std::vector<torch::Tensor*> last = {&s.texture, &s.confidence_value_of_point};
    for (auto& t : per_point_state) last.push_back(&t);
    std::vector<torch::Tensor> src, dst;
    std::vector<vetr_point_array> arrays;
    for (torch::Tensor* t : last)
    {
        if (!t->defined()) continue;
        TORCH_CHECK(t->size(-1) == n && t->element_size() == 4, "RemovePoints: per-point tensors end in the point dimension");
        src.push_back(t->contiguous());
        auto sizes = t->sizes().vec();
        sizes.back() = kept;
        dst.push_back(torch::empty(sizes, t->options()));
        arrays.push_back({src.back().data_ptr(), dst.back().data_ptr(), (int32_t)std::max<int64_t>(src.back().numel() / std::max(n, 1), 1), 1});
    }
    torch::Tensor pos_src = s.t_position.contiguous(), pos_dst = torch::empty({kept, 4}, s.t_position.options());
    arrays.push_back({pos_src.data_ptr(), pos_dst.data_ptr(), 1, 4});
    check(vetr_gather_points(vc, n, kept, new_index.data_ptr<int>(), arrays.data(), (int)arrays.size()), "vetr_gather_points");
    size_t k = 0;
    for (torch::Tensor* t : last)
        if (t->defined()) t->set_(dst[k++]);
    s.t_position.set_(pos_dst);
    if (s.t_index.defined()) s.t_index.set_(torch::arange(kept, s.t_index.options()).reshape({kept, 1}));
    return kept;
}
}  // namespace vetr_torch

// ---------------------------------------------------------------------------------------------------------
// Adding points, ordering a cloud

namespace vetr_torch
{
namespace
{
// t <- cat(t, fill) along the last (point) dimension, in place
void append_columns(torch::Tensor& t, int64_t m, const torch::Tensor& fill_like_values)
{
    if (!t.defined() || m == 0) return;
    t.set_(torch::cat({t.detach(), fill_like_values.to(t.options())}, -1));
}
}  // namespace

int64_t AddNewPoints(RenderScene& s, torch::Tensor new_positions, std::vector<torch::Tensor> per_point_state, bool random_init,
                     torch::Tensor u, torch::Tensor distance)
{
    TORCH_CHECK(s.t_position.defined() && s.t_position.dim() == 2 && s.t_position.size(1) == 4, "AddNewPoints: t_position must be [N,4]");
    TORCH_CHECK(new_positions.dim() == 2 && new_positions.size(1) == 3 && new_positions.dtype() == torch::kFloat32,
                "AddNewPoints: new positions must be [m,3] float");
    torch::NoGradGuard ngg;
    const auto dev  = s.t_position.device();
    const int64_t n = s.t_position.size(0), m = new_positions.size(0), total = n + m;
    auto column_fill = [&](const torch::Tensor& t, double value) {
        auto sizes   = t.sizes().vec();
        sizes.back() = m;
        return torch::full(sizes, value, t.options());
    };
    if (s.texture.defined())
    {
        TORCH_CHECK(s.texture.size(-1) == n, "AddNewPoints: texture does not match the cloud");
        torch::Tensor fill = column_fill(s.texture, 0.5);
        if (random_init) fill = torch::rand_like(fill) * 2 - fill * 2;  // NeuralTexture.cpp:135-138
        append_columns(s.texture, m, fill);
    }
    if (s.confidence_value_of_point.defined()) append_columns(s.confidence_value_of_point, m, column_fill(s.confidence_value_of_point, 0.0));
    for (auto& t : per_point_state)
    {
        if (!t.defined()) continue;
        TORCH_CHECK(t.size(-1) == n, "AddNewPoints: per-point state tensors end in the point dimension");
        append_columns(t, m, column_fill(t, 0.0));
    }
    // positions: appended, then the drop-out radius of the whole cloud as SceneData::ComputeRadius leaves it
    torch::Tensor xyz = torch::cat({s.t_position.detach().slice(1, 0, 3), new_positions.to(dev)}, 0).contiguous();
    if (!distance.defined()) distance = total > 0 ? ComputeRadius(xyz, 4) : torch::empty({0}, xyz.options());
    TORCH_CHECK(distance.numel() == total, "AddNewPoints: one neighbour distance per point");
    if (!u.defined()) u = torch::rand({total}, xyz.options()).clamp_min(1e-12);
    TORCH_CHECK(u.numel() == total, "AddNewPoints: one uniform sample per point");
    const torch::Tensor factor = torch::sqrt(1.0 / u.to(dev, torch::kFloat64)).to(torch::kFloat32);  // d[2] = sqrt(1 / sample)
    const torch::Tensor radius = distance.to(dev, torch::kFloat32).reshape({-1}) * factor.reshape({-1});  // d[3] = d[0] * d[2]
    s.t_position.set_(torch::cat({xyz, radius.reshape({total, 1})}, 1).contiguous());
    if (s.t_index.defined()) s.t_index.set_(torch::arange(total, s.t_index.options()).reshape({total, 1}));
    return total;
}

namespace
{
// spreads the low 21 bits of v so that two zero bits follow every bit
torch::Tensor part1by2(torch::Tensor v)
{
    auto m = [](uint64_t x) { return torch::Scalar((int64_t)x); };
    v = v.bitwise_and(m(0x1FFFFF));
    v = v.bitwise_or(v.bitwise_left_shift(32)).bitwise_and(m(0x1F00000000FFFFull));
    v = v.bitwise_or(v.bitwise_left_shift(16)).bitwise_and(m(0x1F0000FF0000FFull));
    v = v.bitwise_or(v.bitwise_left_shift(8)).bitwise_and(m(0x100F00F00F00F00Full));
    v = v.bitwise_or(v.bitwise_left_shift(4)).bitwise_and(m(0x10C30C30C30C30C3ull));
    v = v.bitwise_or(v.bitwise_left_shift(2)).bitwise_and(m(0x1249249249249249ull));
    return v;
}
}  // namespace

torch::Tensor MortonOrder(torch::Tensor position)
{
    TORCH_CHECK(position.dim() == 2 && position.size(1) >= 3, "MortonOrder: positions must be [N,3] or [N,4]");
    torch::NoGradGuard ngg;
    if (position.size(0) == 0) return torch::empty({0}, torch::TensorOptions().dtype(torch::kLong).device(position.device()));
    const torch::Tensor xyz  = position.detach().slice(1, 0, 3).to(torch::kFloat64);
    const torch::Tensor lo   = std::get<0>(xyz.min(0));
    const torch::Tensor span = (std::get<0>(xyz.max(0)) - lo).clamp_min(1e-12);
    const torch::Tensor q = ((xyz - lo) / span * (double)((1 << 21) - 1)).to(torch::kLong).clamp(0, (1 << 21) - 1);
    const torch::Tensor code = part1by2(q.select(1, 0))
                                   .bitwise_or(part1by2(q.select(1, 1)).bitwise_left_shift(1))
                                   .bitwise_or(part1by2(q.select(1, 2)).bitwise_left_shift(2));
    return std::get<1>(code.sort(/*stable=*/true, 0, false));
}

torch::Tensor RandomBlockShuffle(int64_t n, int64_t block, torch::Tensor block_perm, torch::Device device)
{
    TORCH_CHECK(n >= 0 && block >= 1, "RandomBlockShuffle: bad sizes");
    const int64_t nb = (n + block - 1) / block;
    const auto i64   = torch::TensorOptions().dtype(torch::kLong).device(device);
    if (!block_perm.defined()) block_perm = torch::randperm(nb, i64);
    TORCH_CHECK(block_perm.numel() == nb, "RandomBlockShuffle: one entry per block");
    const torch::Tensor idx = (block_perm.to(device, torch::kLong).reshape({nb, 1}) * block + torch::arange(block, i64).reshape({1, block})).reshape({-1});
    return idx.masked_select(idx < n);
}

torch::Tensor SortBlocksByRadius(torch::Tensor radius, int64_t block)
{
    TORCH_CHECK(radius.dim() == 1 && block >= 1, "SortBlocksByRadius: radius must be [N]");
    torch::NoGradGuard ngg;
    const int64_t n = radius.size(0), nb = n / block;  // the reference sorts full blocks only
    const auto i64  = torch::TensorOptions().dtype(torch::kLong).device(radius.device());
    torch::Tensor perm = torch::arange(n, i64);
    if (nb == 0) return perm;
    const torch::Tensor in_block = std::get<1>(radius.detach().slice(0, 0, nb * block).reshape({nb, block}).sort(/*stable=*/true, 1, false));
    perm.slice(0, 0, nb * block).copy_((in_block + torch::arange(nb, i64).reshape({nb, 1}) * block).reshape({-1}));
    return perm;
}

void ApplyPointOrder(RenderScene& s, torch::Tensor perm, std::vector<torch::Tensor> per_point_state)
{
    TORCH_CHECK(s.t_position.defined() && perm.dim() == 1 && perm.size(0) == s.t_position.size(0), "ApplyPointOrder: one index per point");
    torch::NoGradGuard ngg;
    const int64_t n = perm.size(0);
    perm = perm.to(s.t_position.device(), torch::kLong);
    s.t_position.set_(s.t_position.detach().index_select(0, perm));
    std::vector<torch::Tensor*> last = {&s.texture, &s.confidence_value_of_point};
    for (auto& t : per_point_state) last.push_back(&t);
    for (torch::Tensor* t : last)
    {
        if (!t->defined()) continue;
        TORCH_CHECK(t->size(-1) == n, "ApplyPointOrder: per-point tensors end in the point dimension");
        t->set_(t->detach().index_select(t->dim() - 1, perm.to(t->device())));
    }
    if (s.t_index.defined()) s.t_index.set_(torch::arange(n, s.t_index.options()).reshape({n, 1}));
}
}  // namespace vetr_torch

// ---------------------------------------------------------------------------------------------------------
// Environment map

namespace vetr_torch
{
EnvironmentMapImpl::EnvironmentMapImpl(int channels, int h, int w, bool /*log_texture*/, int axis, int num_images, float inner_radius,
                                       float radius_factor, bool non_subzero_texture)
    : up_axis(axis), channels(channels), non_subzero_texture(non_subzero_texture)
{
    TORCH_CHECK(num_images >= 1 && num_images <= 8, "currently not more spheres are supported");  // EnvironmentMap.cu:97
    const int resolution = std::max(h, w);
    const auto opt = torch::TensorOptions(torch::kCUDA);
    density = register_parameter("density", torch::full({1, 1, num_images, resolution, resolution}, 1.f, opt));
    color   = register_parameter("color", torch::full({1, channels, num_images, resolution, resolution}, 1.f, opt));
    for (int i = 0; i < num_images; ++i) radii.push_back(inner_radius * std::pow(radius_factor, i));  // EnvironmentMap.cu:109-113
}

namespace
{
void fill_env(const EnvironmentSampleState& st, const torch::Tensor& density, const torch::Tensor& color, vetr_envmap& env)
{
    env = vetr_envmap{};
    env.density = density.data_ptr<float>(), env.color = color.data_ptr<float>();
    env.n_spheres = (int)density.size(2), env.resolution = (int)density.size(4), env.channels = (int)color.size(1);
    env.up_axis = st.up_axis, env.non_subzero_texture = st.non_subzero_texture;
    for (int i = 0; i < 8; ++i) env.radii[i] = st.radii[i];
}

std::vector<vetr_view> to_views(const std::vector<ReducedImageInfo>& images)
{
    std::vector<vetr_view> views(images.size());
    for (size_t b = 0; b < images.size(); ++b)
    {
        const ReducedImageInfo& im = images[b];
        vetr_view& v = views[b];
        v = vetr_view{};
        v.w = im.w, v.h = im.h, v.image_index = im.image_index, v.camera_index = im.camera_index, v.camera_model = im.camera_model_type;
        for (int i = 0; i < 5; ++i) v.crop[i] = im.crop_transform[i];
        for (int i = 0; i < 4; ++i) v.rot[i] = im.crop_rotation[i];
    }
    return views;
}
}  // namespace

std::vector<torch::Tensor> EnvironmentMapImpl::Sample2(torch::Tensor poses, torch::Tensor intrinsics,
                                                       const std::vector<ReducedImageInfo>& info_batch, int num_layers,
                                                       const std::vector<std::vector<torch::Tensor>>& layers_cuda)
{
    TORCH_CHECK((int)layers_cuda.size() >= num_layers && !info_batch.empty(), "Sample2: one weight list per layer");
    auto st = torch::make_intrusive<EnvironmentSampleState>();
    st->poses = poses.contiguous(), st->intrinsics = intrinsics.contiguous();
    st->images = info_batch, st->num_layers = num_layers;
    for (int l = 0; l < num_layers; ++l)
    {
        TORCH_CHECK(layers_cuda[l].size() == info_batch.size(), "Sample2: one weight tensor per image and layer");
        // the reference copies every [1,1,h,w] plane into its ray list (EnvironmentMap.cu:423); here into one [B,1,h,w] tensor
        st->weight.push_back(torch::cat(layers_cuda[l], 0).detach().to(torch::kFloat32).contiguous());
    }
    for (size_t i = 0; i < radii.size(); ++i) st->radii[i] = radii[i];
    st->up_axis = up_axis, st->non_subzero_texture = non_subzero_texture, st->cache = &cache_;
    return torch::autograd::EnvironmentSample::apply(density, color, torch::IValue(st));
}
}  // namespace vetr_torch

namespace torch::autograd
{
variable_list EnvironmentSample::forward(AutogradContext* ctx, Variable density, Variable color, IValue state)
{
    using namespace vetr_torch;
    auto st = state.toCustomClass<EnvironmentSampleState>();
    TORCH_CHECK(density.dim() == 5 && color.dim() == 5 && density.is_cuda() && color.is_cuda(), "density / color must be 5-D CUDA tensors");
    c10::cuda::CUDAGuard guard(density.device());
    vetr_ctx* vc = st->cache->context(density.device().index());
    torch::Tensor d = density.detach().contiguous(), c = color.detach().contiguous();
    vetr_envmap env;
    fill_env(*st, d, c, env);
    std::vector<vetr_view> views = to_views(st->images);
    const int B = (int)views.size();
    variable_list out;
    std::vector<const float*> wp;
    std::vector<float*> op;
    int h = views[0].h, w = views[0].w;
    for (int l = 0; l < st->num_layers; ++l, h /= 2, w /= 2)
    {
        TORCH_CHECK(st->weight[l].numel() == (int64_t)B * h * w, "Sample2: weight of layer ", l, " has the wrong size");
        out.push_back(torch::empty({B, env.channels, h, w}, d.options()));
        wp.push_back(st->weight[l].data_ptr<float>());
        op.push_back(out.back().data_ptr<float>());
    }
    vetr_cameras cams{st->poses.data_ptr<double>(), st->intrinsics.data_ptr<float>(), (int)st->poses.size(0), (int)st->intrinsics.size(0)};
    int rc = vetr_envmap_forward(vc, &cams, views.data(), B, st->num_layers, &env, wp.data(), op.data(), st->flags);
    if (rc != VETR_OK) throw std::runtime_error(std::string("vetr_envmap_forward: ") + vetr_strerror(rc));
    ctx->save_for_backward({density, color});
    ctx->saved_data["state"] = state;
    return out;
}

variable_list EnvironmentSample::backward(AutogradContext* ctx, variable_list grad_output)
{
    using namespace vetr_torch;
    auto st    = ctx->saved_data["state"].toCustomClass<EnvironmentSampleState>();
    auto saved = ctx->get_saved_variables();
    torch::Tensor d = saved[0].detach().contiguous(), c = saved[1].detach().contiguous();
    c10::cuda::CUDAGuard guard(d.device());
    vetr_ctx* vc = st->cache->context(d.device().index());
    vetr_envmap env;
    fill_env(*st, d, c, env);
    std::vector<vetr_view> views = to_views(st->images);
    const int B = (int)views.size();
    std::vector<torch::Tensor> g(st->num_layers);
    std::vector<const float*> wp, gp;
    int h = views[0].h, w = views[0].w;
    for (int l = 0; l < st->num_layers; ++l, h /= 2, w /= 2)
    {
        g[l] = grad_output[l].defined() ? grad_output[l].to(torch::kFloat32).contiguous() : torch::zeros({B, env.channels, h, w}, d.options());
        wp.push_back(st->weight[l].data_ptr<float>());
        gp.push_back(g[l].data_ptr<float>());
    }
    torch::Tensor g_density = torch::zeros_like(d), g_color = torch::zeros_like(c);
    vetr_cameras cams{st->poses.data_ptr<double>(), st->intrinsics.data_ptr<float>(), (int)st->poses.size(0), (int)st->intrinsics.size(0)};
    int rc = vetr_envmap_backward(vc, &cams, views.data(), B, st->num_layers, &env, wp.data(), gp.data(),
                                  st->flags | VETR_ENV_NO_DISTORTION_CHECK, g_density.data_ptr<float>(), g_color.data_ptr<float>());
    if (rc != VETR_OK) throw std::runtime_error(std::string("vetr_envmap_backward: ") + vetr_strerror(rc));
    return {g_density, g_color, Variable()};
}
}  // namespace torch::autograd

// ---------------------------------------------------------------------------------------------------------
// Python-visible entry for tests: builds a NeuralRenderInfo from plain arguments and calls BlendPointCloud.
namespace
{
using namespace vetr_torch;

std::vector<torch::Tensor> blend_point_cloud_op(torch::Tensor texture, torch::Tensor background, torch::Tensor position,
                                                torch::Tensor index, torch::Tensor poses_se3, torch::Tensor tangent_poses,
                                                torch::Tensor intrinsics, torch::Tensor confidence, torch::Tensor views_i,
                                                torch::Tensor views_f, int64_t num_layers, int64_t render_mode,
                                                bool output_mask, bool add_depth, bool drop_by_radius, bool use_env_map,
                                                bool need_point_gradient)
{
    static PointRendererCache cache;  // lives as long as the process, like the reference's render-module member
    auto scene = std::make_shared<RenderScene>();
    scene->texture = texture, scene->background_color = background, scene->t_position = position, scene->t_index = index;
    scene->poses_se3 = poses_se3, scene->tangent_poses = tangent_poses, scene->intrinsics = intrinsics;
    scene->confidence_value_of_point = confidence;
    scene->dynamic_refinement_t      = torch::zeros({1}, position.options());
    NeuralRenderInfo info;
    info.scene = scene.get();
    auto vi = views_i.cpu().contiguous();  // [B,5] w h image_index camera_index model
    auto vf = views_f.cpu().contiguous();  // [B,9] crop(5) rot(4)
    for (int64_t b = 0; b < vi.size(0); ++b)
    {
        ReducedImageInfo im;
        const int* pi   = vi.data_ptr<int>() + 5 * b;
        const float* pf = vf.data_ptr<float>() + 9 * b;
        im.w = pi[0], im.h = pi[1], im.image_index = pi[2], im.camera_index = pi[3], im.camera_model_type = pi[4];
        for (int i = 0; i < 5; ++i) im.crop_transform[i] = pf[i];
        for (int i = 0; i < 4; ++i) im.crop_rotation[i] = pf[5 + i];
        info.images.push_back(im);
    }
    info.params.num_texture_channels      = (int)texture.size(0);
    info.params.render_mode               = (int)render_mode;
    info.params.dropout                   = 0.f;
    info.params.output_background_mask    = output_mask;
    info.params.add_depth_to_network      = add_depth;
    info.params.drop_out_points_by_radius = drop_by_radius;
    info.params.use_environment_map       = use_env_map;
    info.params.need_point_gradient       = need_point_gradient;
    info.num_layers = (int)num_layers;
    info.cache      = &cache;
    // the scene must outlive the autograd graph: keep it in a holder that the returned tensors do not own; tests call
    // backward before the next forward, so a static slot is enough here
    static std::shared_ptr<RenderScene> keep;
    keep       = scene;
    info.scene = keep.get();
    return BlendPointCloud(&info);
}

// FillSceneGridWithLoss for one view given as the same integer / float rows as blend_point_cloud's views
void fill_scene_grid_with_loss_op(torch::Tensor poses_se3, torch::Tensor intrinsics, torch::Tensor view_i, torch::Tensor view_f,
                                  torch::Tensor cell_bb_min, torch::Tensor cell_bb_length, torch::Tensor cell_value,
                                  torch::Tensor cell_access_count, torch::Tensor loss_img)
{
    static PointRendererCache cache;
    RenderScene scene;
    scene.poses_se3 = poses_se3, scene.intrinsics = intrinsics;
    scene.t_cell_bb_min = cell_bb_min, scene.t_cell_bb_length = cell_bb_length;
    scene.t_cell_value = cell_value, scene.t_cell_access_count = cell_access_count;
    auto vi = view_i.cpu().contiguous();
    auto vf = view_f.cpu().contiguous();
    ReducedImageInfo im;
    const int* pi   = vi.data_ptr<int>();
    const float* pf = vf.data_ptr<float>();
    im.w = pi[0], im.h = pi[1], im.image_index = pi[2], im.camera_index = pi[3], im.camera_model_type = pi[4];
    for (int i = 0; i < 5; ++i) im.crop_transform[i] = pf[i];
    for (int i = 0; i < 4; ++i) im.crop_rotation[i] = pf[5 + i];
    cache.FillSceneGridWithLoss(0, scene, {im}, loss_img);
}

// EnvironmentMap::Sample2 with the caller's parameter tensors (density [1,1,S,R,R], color [1,C,S,R,R]) and one
// transmittance tensor [B,1,h_l,w_l] per layer; views as in blend_point_cloud.
std::vector<torch::Tensor> environment_map_sample2_op(torch::Tensor density, torch::Tensor color, double inner_radius,
                                                      double radius_factor, int64_t up_axis, bool non_subzero_texture,
                                                      torch::Tensor poses_se3, torch::Tensor intrinsics, torch::Tensor views_i,
                                                      torch::Tensor views_f, int64_t num_layers, std::vector<torch::Tensor> weights)
{
    // the module outlives the autograd graph of the call (its cache owns the context the backward node uses)
    static std::vector<EnvironmentMap> keep;
    EnvironmentMap env((int)color.size(1), 1, 1, false, (int)up_axis, (int)density.size(2), (float)inner_radius, (float)radius_factor,
                       non_subzero_texture);
    keep.push_back(env);
    if (keep.size() > 8) keep.erase(keep.begin());
    env->density = density, env->color = color;
    auto vi = views_i.cpu().contiguous();
    auto vf = views_f.cpu().contiguous();
    std::vector<ReducedImageInfo> images;
    for (int64_t b = 0; b < vi.size(0); ++b)
    {
        ReducedImageInfo im;
        const int* pi   = vi.data_ptr<int>() + 5 * b;
        const float* pf = vf.data_ptr<float>() + 9 * b;
        im.w = pi[0], im.h = pi[1], im.image_index = pi[2], im.camera_index = pi[3], im.camera_model_type = pi[4];
        for (int i = 0; i < 5; ++i) im.crop_transform[i] = pf[i];
        for (int i = 0; i < 4; ++i) im.crop_rotation[i] = pf[5 + i];
        images.push_back(im);
    }
    std::vector<std::vector<torch::Tensor>> layers(num_layers);
    for (int64_t l = 0; l < num_layers; ++l)
        for (int64_t b = 0; b < vi.size(0); ++b) layers[l].push_back(weights[l].slice(0, b, b + 1));
    return env->Sample2(poses_se3, intrinsics, images, (int)num_layers, layers);
}
}  // namespace

TORCH_LIBRARY(vetr, m)
{
    m.def("fill_scene_grid_with_loss", &fill_scene_grid_with_loss_op);
    m.class_<vetr_torch::EnvironmentSampleState>("EnvironmentSampleState").def(torch::init());
    m.def("environment_map_sample2", &environment_map_sample2_op);
    m.def("remove_points", [](torch::Tensor texture, torch::Tensor confidence, torch::Tensor position, torch::Tensor index,
                              torch::Tensor indices_to_remove, std::vector<torch::Tensor> state) {
        vetr_torch::RenderScene scene;
        scene.texture = texture, scene.confidence_value_of_point = confidence, scene.t_position = position, scene.t_index = index;
        return vetr_torch::RemovePoints(scene, indices_to_remove, state);  // the tensors shrink in place
    });
    m.def("compute_radius", [](torch::Tensor position, int64_t n) { return vetr_torch::ComputeRadius(position, (int)n); });
    m.def("add_new_points", [](torch::Tensor texture, torch::Tensor confidence, torch::Tensor position, torch::Tensor index,
                               torch::Tensor new_positions, std::vector<torch::Tensor> state, bool random_init,
                               c10::optional<torch::Tensor> u, c10::optional<torch::Tensor> distance) {
        vetr_torch::RenderScene scene;
        scene.texture = texture, scene.confidence_value_of_point = confidence, scene.t_position = position, scene.t_index = index;
        return vetr_torch::AddNewPoints(scene, new_positions, state, random_init, u.value_or(torch::Tensor()),
                                        distance.value_or(torch::Tensor()));  // the tensors grow in place
    });
    m.def("morton_order", &vetr_torch::MortonOrder);
    m.def("random_block_shuffle", [](int64_t n, int64_t block, c10::optional<torch::Tensor> block_perm) {
        const torch::Tensor bp = block_perm.value_or(torch::Tensor());
        return vetr_torch::RandomBlockShuffle(n, block, bp, bp.defined() ? bp.device() : torch::Device(torch::kCPU));
    });
    m.def("sort_blocks_by_radius", &vetr_torch::SortBlocksByRadius);
    m.def("apply_point_order", [](torch::Tensor texture, torch::Tensor confidence, torch::Tensor position, torch::Tensor index,
                                  torch::Tensor perm, std::vector<torch::Tensor> state) {
        vetr_torch::RenderScene scene;
        scene.texture = texture, scene.confidence_value_of_point = confidence, scene.t_position = position, scene.t_index = index;
        vetr_torch::ApplyPointOrder(scene, perm, state);  // the tensors are reordered in place
    });
    m.class_<vetr_torch::NeuralRenderInfo>("NeuralRenderInfo").def(torch::init());
    m.def("blend_point_cloud", &blend_point_cloud_op);
    m.def("apply_tangent_to_pose", &vetr_torch::ApplyTangentToPose);
}
