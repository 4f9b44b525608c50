// C++/libtorch host side of the rasterizer: the reference's operator surface on top of the C ABI (include/vetr.h).
//
// Mirrors, with the same names, argument order and return layout:
//   NeuralRenderInfo                      rendering/PointRenderer.h:23-34
//   torch::autograd::PointRender          rendering/PointRenderer.h:39-47, rendering/RenderInfo.cpp:32-67
//   BlendPointCloud(NeuralRenderInfo*)    rendering/PointRenderer.h:53,   rendering/RenderInfo.cpp:18-30
//   ApplyTangentToPose(tangent, pose)     rendering/PointRenderer.h:64,   rendering/PointRenderer.cu:1343-1349
//   PointRendererCache / LayerCuda        rendering/PointRenderer.h:66-248 (the members outside code reads:
//                                         layers_cuda[i].weight / .depth, num_batches, render_mode)
//   PointRendererCache::FillSceneGridWithLoss   rendering/PointRenderer.h:152, RenderForward.cu:761-791
//   EnvironmentMapImpl (constructor, density, color, Sample2)   rendering/EnvironmentMap.h:252-301
//   SceneData::ComputeRadius(point_cloud, n)   data/SceneData.h:396
//   NeuralScene::RemovePoints(indices_to_remove)   data/NeuralScene.h (device part)
//   NeuralScene::AddNewPoints(positions)           data/NeuralScene.cpp:1013-1074 (device part)
//   ReorderMorton64 / RandomBlockShuffle / SortBlocksByRadius   data/SceneData.cpp:105-108
// The reference's NeuralScene / RenderParams / ReducedImageInfo come from parts of VET that need the saiga library;
// the structs below carry exactly the fields the render operator reads from them, under the same names, so that the
// reference's call site (models/Pipeline.cpp:133 via RenderModule.cpp:45-245) maps onto them one to one.
#pragma once
#include <torch/torch.h>

#include <memory>
#include <vector>

#include "../../include/vetr.h"

namespace vetr_torch
{
// data/SceneData.h:39-50
struct ReducedImageInfo
{
    int w = 0, h = 0;
    int image_index       = -1;
    int camera_index      = -1;
    int camera_model_type = 0;                    // CameraModel::PINHOLE_DISTORTION
    float crop_transform[5] = {1, 1, 0, 0, 0};    // IntrinsicsPinholef: fx fy cx cy s
    float crop_rotation[4]  = {1, 0, 0, 1};       // row-major 2x2
};

// data/Settings.h:19-73 (fields the operator reads)
struct RenderParams
{
    bool check_normal               = false;
    float dropout                   = 0.25f;
    float depth_accept              = 0.01f;
    float depth_accept_blend        = 0.01f;
    bool ghost_gradients            = false;
    float drop_out_radius_threshold = 0.6f;
    bool drop_out_points_by_radius  = true;
    float distortion_gradient_factor = 0.005f;
    float K_gradient_factor          = 0.5f;
    int num_texture_channels         = 4;
    float dist_cutoff                = 20.f;
    bool output_background_mask      = false;
    float output_background_mask_value = 0.f;
    bool add_depth_to_network        = false;
    float stability_cutoff_value     = 10000.f;
    bool need_point_gradient         = true;
    bool use_environment_map         = true;
    int render_mode                  = 1;
    bool viewer_only                 = false;
    int debug_max_list_length        = -1;
};

// The tensors of NeuralScene the operator reads (data/NeuralScene.h:22-121): texture->texture,
// texture->background_color, texture->confidence_value_of_point, point_cloud_cuda->t_position / t_index,
// poses->poses_se3 / tangent_poses, intrinsics->intrinsics.
struct RenderScene
{
    torch::Tensor texture;                    // [C,N] f32
    torch::Tensor background_color;           // [C]
    torch::Tensor confidence_value_of_point;  // [1,N]
    torch::Tensor t_position;                 // [N,4]
    torch::Tensor t_index;                    // [N,1] i32
    torch::Tensor poses_se3;                  // [n,8] f64
    torch::Tensor tangent_poses;              // [n,6] f64
    torch::Tensor intrinsics;                 // [n_cam,13]
    torch::Tensor dynamic_refinement_t;       // dummy [1] (models/Pipeline.cpp:128)
    // scene grid of the error tomography (NeuralPointCloudCuda.h:100-106); only FillSceneGridWithLoss reads them
    torch::Tensor t_cell_bb_min, t_cell_bb_length;  // [n_cells,3] f32
    torch::Tensor t_cell_value;                     // [n_cells,1] f32
    torch::Tensor t_cell_access_count;              // [n_cells,1] i32
};

struct LayerCuda
{
    int w = 0, h = 0;
    torch::Tensor depth;   // [B,1,h,w] nearest depth, 100000 where empty
    torch::Tensor weight;  // [B,1,h,w] final transmittance
};

class PointRendererCache
{
   public:
    ~PointRendererCache();
    enum RenderMode
    {
        FUZZY_DT       = 0,
        FULL_BLEND     = 1,
        FUZZY_BLEND    = 2,
        BILINEAR_BLEND = 3,
    } render_mode = FULL_BLEND;
    std::vector<LayerCuda> layers_cuda;
    int num_batches = 0;
    torch::Tensor dropout_points;  // [B,N] (1 = dropped), kept for inspection like the reference's member

    vetr_ctx* context(int device);  // one C-ABI context per cache, created on first use on the current stream

    // Fragment buffer sizing.  The reference reads the list sizes back (two blocking .item() per view and level,
    // PointRenderer.cu:796-822) and allocates exactly; here nothing is read back inside a call.  The first call for a
    // scene shape uses the bound that cannot overflow (vetr_list_capacity: every point on every level); every call copies
    // its status words (fragment total, overflow flag) to pinned host memory behind its kernels, and later calls size the
    // buffer as kFragmentHeadroom x the largest total per view seen so far.  The words of earlier calls are looked at when
    // the next call starts and again before a backward pass (long after the copy finished, so nothing stalls): an overflow
    // or a list the mode-2 backward pass had to skip raises an error there, and the next call is sized by the safe bound.
    static constexpr double kFragmentHeadroom = 1.5;
    int64_t FragmentCapacity(int64_t safe_bound, int n_views, int n_points, int num_layers, int w, int h, int mode);
    void NoteStatus(const torch::Tensor& status_dev, int64_t capacity, int n_views, bool after_backward);
    void CheckEarlierCalls();  // throws std::runtime_error
    int64_t last_fragment_capacity = 0;  // records the buffer of the most recent forward group held (for reporting)

    // PointRendererCache::FillSceneGridWithLoss (RenderForward.cu:761-791, called from train.cpp:1077): adds the loss image
    // of images[batch] ([C,h,w]) to the grid cells of `scene` that its camera sees.  Enqueued on the current stream; the
    // reference synchronises the device afterwards, this does not.
    void FillSceneGridWithLoss(int batch, RenderScene& scene, const std::vector<ReducedImageInfo>& images,
                               torch::Tensor loss_img, float dist_cutoff = 20.f);

   private:
    vetr_ctx* ctx_ = nullptr;
    int device_    = -1;
    struct Pending
    {
        int slot;  // of status_host_ / status_event_
        int64_t capacity;
        int n_views;
        bool after_backward;
    };
    static constexpr size_t kStatusSlots = 16;
    std::vector<Pending> pending_;
    int* status_host_ = nullptr;  // [kStatusSlots][4] pinned: {fragment total, flags, longest list, work items} of a call
    CUevent_st* status_event_[kStatusSlots] = {};  // cudaEvent_t recorded behind the copy into the slot
    int64_t high_water_per_view_ = 0;  // largest fragment total per view seen for shape_
    int64_t shape_[5]            = {-1, -1, -1, -1, -1};
};

class NeuralRenderInfo : public torch::CustomClassHolder
{
   public:
    RenderScene* scene = nullptr;
    std::vector<ReducedImageInfo> images;
    RenderParams params;
    int num_layers    = 4;
    bool train        = true;
    int current_epoch = 0;
    PointRendererCache* cache = nullptr;
};

// Render the scene into a batch of images; every image is a pyramid of layers.  Returns num_layers colour tensors
// [B,C,h_l,w_l], then num_layers depth tensors if add_depth_to_network, then num_layers masks [B,1,h_l,w_l] if
// output_background_mask (rendering/RenderInfo.cpp:40-42, RenderModule.cpp:74-102).
std::vector<torch::Tensor> BlendPointCloud(NeuralRenderInfo* info);

void ApplyTangentToPose(torch::Tensor tangent, torch::Tensor pose);

// SceneData::ComputeRadius (data/SceneData.h:396, SceneData.cpp:554-597) for a cloud that already lives on the GPU:
// position [N,3] or [N,4] float CUDA tensor -> [N] distances to the n-th nearest other point (the reference's data[i](0)).
torch::Tensor ComputeRadius(torch::Tensor position, int n = 4);

// NeuralScene::RemovePoints (data/NeuralScene.cpp:1156-1239) for the tensors the render operator reads, without the host
// round trip: t_position and t_index (rebuilt as the identity, as the reference's cloud constructor does), texture and
// confidence_value_of_point shrink in place (Tensor::set_, as RemoveAndFlatten does, so parameters keep their identity),
// and so does every tensor of `per_point_state` whose last dimension is the point count (the optimizer's exp_avg /
// exp_avg_sq, my_adam.cpp:107-135).  indices_to_remove: int64, any device.  Returns the number of points left.
int64_t RemovePoints(RenderScene& scene, torch::Tensor indices_to_remove, std::vector<torch::Tensor> per_point_state = {});

// NeuralScene::AddNewPoints (data/NeuralScene.cpp:1013-1074) for the tensors the render operator reads, on whatever device
// they live: the new positions are appended behind the existing ones (SceneData::AddPoints, SceneData.cpp:669-691),
// t_index is rebuilt as the identity, texture gets columns of 0.5 - or of U(-1, 1) with `random_init` - and
// confidence_value_of_point columns of 0 (NeuralPointTextureImpl::EnlargeTexture / ResizeAndFill, NeuralTexture.h:94-103,
// NeuralTexture.cpp:118-158), every tensor of `per_point_state` (the optimizer's exp_avg / exp_avg_sq,
// MyAdam::appendToInternalState, my_adam.cpp:137-170) columns of 0; all in place (Tensor::set_), so parameters keep
// their identity.  The reference then recomputes the drop-out radius of the WHOLE cloud (ComputeRadius inside AddPoints):
// column 3 of t_position becomes distance to the 4th nearest other point x sqrt(1 / u).  `u`: [N + m] uniform samples in
// (0, 1] (drawn with torch::rand when undefined; the reference draws them from its own generator).  `distance`: the
// neighbour distances [N + m] if the caller has them; otherwise they come from ComputeRadius (CUDA tensors).
// Returns the new number of points.
int64_t AddNewPoints(RenderScene& scene, torch::Tensor new_positions, std::vector<torch::Tensor> per_point_state = {},
                     bool random_init = false, torch::Tensor u = {}, torch::Tensor distance = {});

// The ordering the reference gives a cloud when a scene is prepared (data/SceneData.cpp:105-108: ReorderMorton64,
// RandomBlockShuffle(256), ComputeRadius, SortBlocksByRadius(256)), as permutations computed with libtorch operators on
// the tensors' own device (torch's sort is a device radix sort on CUDA tensors), so that texture and optimizer state can
// follow the positions.  Each function returns int64 indices: element i of the new order is element perm[i] of the old.
//   MortonOrder          stable ascending order of the 63-bit Morton code of the positions (21 bits per axis over the
//                        bounding box, x in the lowest bit of every triple)
//   RandomBlockShuffle   whole blocks of `block` consecutive points in the order `block_perm` (a permutation of the
//                        ceil(n / block) block indices; torch::randperm when undefined); a shorter last block moves as it is
//   SortBlocksByRadius   inside every full block, ascending by radius (SceneData.cpp:1005-1018; the tail stays)
//   ApplyPointOrder      reorders t_position, texture, confidence_value_of_point and `per_point_state` in place and
//                        rebuilds t_index as the identity
torch::Tensor MortonOrder(torch::Tensor position);
torch::Tensor RandomBlockShuffle(int64_t n, int64_t block, torch::Tensor block_perm, torch::Device device);
torch::Tensor SortBlocksByRadius(torch::Tensor radius, int64_t block);
void ApplyPointOrder(RenderScene& scene, torch::Tensor perm, std::vector<torch::Tensor> per_point_state = {});

// What one Sample2 call hands to its autograd node.
struct EnvironmentSampleState : public torch::CustomClassHolder
{
    torch::Tensor poses, intrinsics;
    std::vector<ReducedImageInfo> images;
    std::vector<torch::Tensor> weight;  // per layer [B,1,h,w]
    int num_layers = 0, flags = 0;
    float radii[8] = {};
    int up_axis = 0;
    bool non_subzero_texture = false;
    PointRendererCache* cache = nullptr;
};

// rendering/EnvironmentMap.h:252-301.  Same constructor arguments, parameters and Sample2 result; `scene` (only read
// for OCam cameras) and the timer are not taken.  density / color receive gradients through autograd as in the
// reference, where forward_mps5 is built from differentiable libtorch operators.
class EnvironmentMapImpl : public torch::nn::Module
{
   public:
    EnvironmentMapImpl(int channels, int h, int w, bool log_texture, int axis = 0, int num_images = 4, float inner_radius = 20.f,
                       float radius_factor = 5.f, bool non_subzero_texture = false);

    // layers_cuda[layer][batch]: the rasterizer's transmittance of that image and layer, [1,1,h_l,w_l]
    // (RenderModule.cpp:133-141).  Returns per layer [B,channels,h_l,w_l].
    std::vector<torch::Tensor> Sample2(torch::Tensor poses, torch::Tensor intrinsics, const std::vector<ReducedImageInfo>& info_batch,
                                       int num_layers, const std::vector<std::vector<torch::Tensor>>& layers_cuda);

    torch::Tensor density;  // [1, 1, num_images, resolution, resolution]
    torch::Tensor color;    // [1, channels, num_images, resolution, resolution]
    int NumImages() { return (int)density.size(2); }

   private:
    std::vector<float> radii;
    int up_axis;
    int channels;
    bool non_subzero_texture;
    PointRendererCache cache_;  // owns the C-ABI context
};
TORCH_MODULE(EnvironmentMap);
}  // namespace vetr_torch

namespace torch::autograd
{
struct PointRender : public Function<PointRender>
{
    static variable_list forward(AutogradContext* ctx, Variable texture, Variable background_color, Variable points,
                                 Variable pose_tangents, Variable intrinsics, Variable confidence,
                                 Variable dynamic_refinement, IValue info);
    static variable_list backward(AutogradContext* ctx, variable_list grad_output);
};

struct EnvironmentSample : public Function<EnvironmentSample>
{
    static variable_list forward(AutogradContext* ctx, Variable density, Variable color, IValue state);
    static variable_list backward(AutogradContext* ctx, variable_list grad_output);
};
}  // namespace torch::autograd
