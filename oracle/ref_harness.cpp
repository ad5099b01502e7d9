// Harness around the reference's own CUDA build of the training-step path.
//
// TEST INFRASTRUCTURE, not product. This translation unit is compiled together with the UNMODIFIED
// reference sources (gsplat/*.cu|cpp, src/training/kernels/{ssim,regularization}.cu,
// src/training/fastgs/{optimizer,rasterization}/src/*.cu, src/training/rasterization/
// {rasterizer_autograd,fast_rasterizer_autograd}.cpp, src/training/optimizers/{fused_adam,scheduler}.cpp),
// which are read where they lie in the reference checkout and never copied, into one Python extension
// module. It serves two purposes: (1) the checker that the CUDA library of this repository and the CPU
// oracle are compared with, and (2) the timed comparator of the benchmark's reference arm. It never loads
// or calls the library of this repository.
//
// Two kinds of entry points:
//   * the reference's operators bound one to one (namespace gsplat of gsplat/Ops.h:12-270, fusedssim /
//     fusedssim_backward of src/training/kernels/ssim.cu:431/:476, fused_ssim of
//     include/kernels/fused_ssim.cuh:117, adam_step_wrapper of fastgs/optimizer/src/adam_api.cu:8,
//     forward_wrapper / backward_wrapper of fastgs/rasterization/src/rasterization_api.cu:16/:92, the two
//     regularizers of src/training/kernels/regularization.cu);
//   * RefTrainer, which drives one training step with the reference's own autograd nodes
//     (FusedRasterizationWithSHFunction, FastGSRasterize, _FusedSSIM) and its own FusedAdam /
//     ExponentialLR classes. Only the pieces of host glue that depend on the reference's Camera /
//     SplatData classes (whose translation units need the whole application) are restated here on plain
//     tensors, each with the reference lines it follows.
#include <torch/extension.h>

#include <cmath>
#include <memory>
#include <optional>
#include <tuple>
#include <vector>

#include "Ops.h"
#include "adam_api.h"
#include "kernels/fused_ssim.cuh"
#include "kernels/regularization.cuh"
#include "optimizers/fused_adam.hpp"
#include "optimizers/scheduler.hpp"
#include "rasterization/fast_rasterizer_autograd.hpp"
#include "rasterization/rasterizer.hpp"
#include "rasterization/rasterizer_autograd.hpp"
#include "rasterization_api.h"

namespace {

    using torch::Tensor;
    using OptTensor = std::optional<Tensor>;
    using torch::indexing::None;
    using torch::indexing::Slice;

    // None -> the reference's defaults (gsplat/Cameras.h:27-45); otherwise a sequence (alpha, beta, kappa,
    // in_image_margin_factor, require_all_sigma_points_valid).
    UnscentedTransformParameters ut_from(const py::object& o) {
        UnscentedTransformParameters ut{};
        if (o.is_none())
            return ut;
        auto t = o.cast<std::vector<double>>();
        TORCH_CHECK(t.size() == 5, "ut_params: five values");
        ut.alpha = float(t[0]);
        ut.beta = float(t[1]);
        ut.kappa = float(t[2]);
        ut.in_image_margin_factor = float(t[3]);
        ut.require_all_sigma_points_valid = t[4] != 0.0;
        return ut;
    }

    // ------------------------------------------------------------------------------------------
    // The training step, in the order of Trainer::train_step (src/training/trainer.cpp:599-790).
    // ------------------------------------------------------------------------------------------
    struct RefRender {
        Tensor image; // [3, H, W] clamped to [0, 1] on the gut path
        Tensor alpha; // [1, H, W]
        Tensor depth;
        Tensor radii;   // [C, N, 2] (gut path)
        Tensor means2d; // [C, N, 2]
        Tensor depths;  // [C, N]
    };

    class RefTrainer {
    public:
        // Raw SplatData tensors (src/core/splat_data.hpp:104-109): means [N,3], sh0 [N,1,3], shN [N,K-1,3],
        // scaling_raw [N,3] (log), rotation_raw [N,4] (wxyz), opacity_raw [N,1] (logit).
        // Optimizer set-up of MCMC::initialize (src/training/strategies/mcmc.cpp:451-497): six groups in this
        // order, eps 1e-15, betas (0.9, 0.999), exponential decay of group 0 to 1 % over `iterations`.
        RefTrainer(Tensor means, Tensor sh0, Tensor shN, Tensor scaling_raw, Tensor rotation_raw, Tensor opacity_raw,
                   std::vector<double> lrs, int iterations, int active_sh_degree)
            : sh_degree_(active_sh_degree) {
            TORCH_CHECK(lrs.size() == 6, "six learning rates: means, sh0, shN, scaling, rotation, opacity");
            auto leaf = [](const Tensor& t) { return t.detach().clone().contiguous().set_requires_grad(true); };
            means_ = leaf(means);
            sh0_ = leaf(sh0);
            shN_ = leaf(shN);
            scaling_ = leaf(scaling_raw);
            rotation_ = leaf(rotation_raw);
            opacity_ = leaf(opacity_raw);
            densification_info_ = torch::empty({0});

            using Options = gs::training::FusedAdam::Options;
            std::vector<torch::optim::OptimizerParamGroup> groups;
            auto add_param_group = [&groups](const Tensor& param, double lr) {
                auto options = std::make_unique<Options>(lr);
                options->eps(1e-15).betas(std::make_tuple(0.9, 0.999));
                groups.emplace_back(std::vector<Tensor>{param},
                                    std::unique_ptr<torch::optim::OptimizerOptions>(std::move(options)));
            };
            add_param_group(means_, lrs[0]);
            add_param_group(sh0_, lrs[1]);
            add_param_group(shN_, lrs[2]);
            add_param_group(scaling_, lrs[3]);
            add_param_group(rotation_, lrs[4]);
            add_param_group(opacity_, lrs[5]);
            auto global_options = std::make_unique<Options>(0.f);
            global_options->eps(1e-15);
            optimizer_ = std::make_unique<gs::training::FusedAdam>(std::move(groups), std::move(global_options));
            const double gamma = std::pow(0.01, 1.0 / iterations);
            scheduler_ = std::make_unique<gs::training::ExponentialLR>(*optimizer_, gamma, 0);
        }

        // rasterize() of src/training/rasterization/rasterizer.cpp:15-225 on plain tensors: activations of
        // SplatData (src/core/splat_data.cpp:267-286), the fused autograd node, the clamp / permute of the
        // outputs. viewmat [1,4,4] world-to-camera, K [1,3,3].
        RefRender rasterize(const Tensor& viewmat, const Tensor& K, int width, int height, const Tensor& bg_color,
                            float scaling_modifier, bool antialiased, int render_mode, int camera_model,
                            const OptTensor& radial, const OptTensor& tangential) {
            auto means3D = means_;
            auto opacities = torch::sigmoid(opacity_).squeeze(-1);
            auto scales = torch::exp(scaling_);
            auto rotations = torch::nn::functional::normalize(
                rotation_, torch::nn::functional::NormalizeFuncOptions().dim(-1));
            auto sh_coeffs = torch::cat({sh0_, shN_}, 1);

            Tensor prepared_bg_color;
            if (bg_color.defined() && bg_color.numel() > 0)
                prepared_bg_color = bg_color.view({1, -1});

            auto settings = gs::training::FusedRasterizationSettings{
                width, height, 16, 0.3f, 0.01f, 10000.0f, 0.0f, scaling_modifier, antialiased,
                static_cast<gsplat::CameraModelType>(camera_model), static_cast<gs::training::RenderMode>(render_mode)};
            auto ut_params = UnscentedTransformParameters{};

            auto out = gs::training::FusedRasterizationWithSHFunction::apply(
                means3D, rotations, scales, opacities, sh_coeffs, sh_degree_,
                prepared_bg_color.defined() ? prepared_bg_color
                                            : torch::tensor({0.0f, 0.0f, 0.0f}, means3D.options()),
                std::nullopt, viewmat, K, radial, tangential, std::nullopt, settings, ut_params);

            auto rendered_image = out[0];
            auto rendered_alpha = out[1];
            Tensor final_image, final_depth;
            switch (render_mode) {
            case 0: final_image = rendered_image; break;
            case 1: final_depth = rendered_image; break;
            case 2: final_depth = rendered_image / rendered_alpha.clamp_min(1e-10); break;
            case 3:
                final_image = rendered_image.index({Slice(), Slice(), Slice(), Slice(None, -1)});
                final_depth = rendered_image.index({Slice(), Slice(), Slice(), Slice(-1, None)});
                break;
            default: {
                final_image = rendered_image.index({Slice(), Slice(), Slice(), Slice(None, -1)});
                auto accum = rendered_image.index({Slice(), Slice(), Slice(), Slice(-1, None)});
                final_depth = accum / rendered_alpha.clamp_min(1e-10);
            }
            }
            RefRender r;
            if (final_image.defined() && final_image.numel() > 0)
                r.image = torch::clamp(final_image.squeeze(0).permute({2, 0, 1}), 0.0f, 1.0f);
            r.alpha = rendered_alpha.squeeze(0).permute({2, 0, 1});
            if (final_depth.defined() && final_depth.numel() > 0)
                r.depth = final_depth.squeeze(0).permute({2, 0, 1});
            r.radii = out[2];
            r.means2d = out[3];
            r.depths = out[4];
            return r;
        }

        // fast_rasterize() of src/training/rasterization/fast_rasterizer.cpp:13-71 on plain tensors. The
        // camera position is the translation column of the inverse pose (src/core/camera.cpp:55-56).
        RefRender fast_rasterize(const Tensor& w2c, float fx, float fy, float cx, float cy, int width, int height,
                                 const Tensor& bg_color) {
            fast_gs::rasterization::FastGSSettings settings;
            auto c2w = torch::inverse(w2c.squeeze());
            settings.cam_position = c2w.index({Slice(None, 3), 3}).contiguous().squeeze();
            settings.active_sh_bases = (sh_degree_ + 1) * (sh_degree_ + 1);
            settings.width = width;
            settings.height = height;
            settings.focal_x = fx;
            settings.focal_y = fy;
            settings.center_x = cx;
            settings.center_y = cy;
            settings.near_plane = 0.01f;
            settings.far_plane = 1e10f;
            auto out = gs::training::FastGSRasterize::apply(means_, scaling_, rotation_, opacity_, sh0_, shN_, w2c,
                                                            densification_info_, settings);
            RefRender r;
            r.image = out[0];
            r.alpha = out[1];
            r.image = r.image + (1.0f - r.alpha) * bg_color.unsqueeze(-1).unsqueeze(-1);
            return r;
        }

        // compute_photometric_loss of src/training/trainer.cpp:107-134.
        static Tensor photometric_loss(const Tensor& image, const Tensor& gt_image, float lambda_dssim) {
            Tensor rendered = image.dim() == 3 ? image.unsqueeze(0) : image;
            Tensor gt = gt_image.dim() == 3 ? gt_image.unsqueeze(0) : gt_image;
            TORCH_CHECK(rendered.sizes() == gt.sizes(), "size mismatch");
            auto l1_loss = torch::l1_loss(rendered, gt);
            auto ssim_loss = 1.f - fused_ssim(rendered, gt, "valid", /*train=*/true);
            return (1.f - lambda_dssim) * l1_loss + lambda_dssim * ssim_loss;
        }

        // Forward + loss + backward of one camera; gradients are left in .grad of the six leaves.
        std::tuple<Tensor, Tensor, Tensor> forward_backward(bool gut, const Tensor& viewmat, const Tensor& K, int width,
                                                            int height, const Tensor& bg_color, const Tensor& gt_image,
                                                            float lambda_dssim) {
            RefRender r = render(gut, viewmat, K, width, height, bg_color);
            Tensor loss = photometric_loss(r.image, gt_image, lambda_dssim);
            loss.backward();
            return {r.image.detach(), r.alpha.detach(), loss.detach()};
        }

        // One iteration of Trainer::train_step (trainer.cpp:672-700, :761-772) for the photometric loss:
        // render, loss, backward, the loss read back to the host (loss.item<float>(), trainer.cpp:698), the two
        // regularizers when their weights are positive (trainer.cpp:700-712), then MCMC::step
        // (mcmc.cpp:395-402): FusedAdam::step, zero_grad(set_to_none), scheduler step.
        float train_step(int iter, bool gut, const Tensor& viewmat, const Tensor& K, int width, int height,
                         const Tensor& bg_color, const Tensor& gt_image, float lambda_dssim, float scale_reg,
                         float opacity_reg) {
            RefRender r = render(gut, viewmat, K, width, height, bg_color);
            Tensor loss = photometric_loss(r.image, gt_image, lambda_dssim);
            loss.backward();
            float loss_value = loss.item<float>();
            if (scale_reg > 0.0f)
                loss_value += gs::regularization::compute_exp_l1_regularization_with_grad_cuda(scaling_, scale_reg);
            if (opacity_reg > 0.0f)
                loss_value += gs::regularization::compute_sigmoid_l1_regularization_with_grad_cuda(opacity_, opacity_reg);
            {
                torch::NoGradGuard no_grad;
                optimizer_->step(iter);
                optimizer_->zero_grad(true, iter);
                scheduler_->step();
            }
            return loss_value;
        }

        // Forward only (no autograd graph), for the forward-only workloads.
        RefRender render_no_grad(bool gut, const Tensor& viewmat, const Tensor& K, int width, int height,
                                 const Tensor& bg_color, int camera_model) {
            torch::NoGradGuard no_grad;
            if (gut)
                return rasterize(viewmat, K, width, height, bg_color, 1.0f, false, 0, camera_model, std::nullopt,
                                 std::nullopt);
            return render(false, viewmat, K, width, height, bg_color);
        }

        void optimizer_step(int iter) {
            torch::NoGradGuard no_grad;
            optimizer_->step(iter);
            optimizer_->zero_grad(true, iter);
            scheduler_->step();
        }

        std::vector<Tensor> params() const { return {means_, sh0_, shN_, scaling_, rotation_, opacity_}; }
        std::vector<Tensor> grads() const {
            std::vector<Tensor> g;
            for (const auto& p : params())
                g.push_back(p.grad().defined() ? p.grad() : Tensor());
            return g;
        }
        // (exp_avg, exp_avg_sq, step_count) of each group, empty tensors before the first step.
        std::vector<std::tuple<Tensor, Tensor, int64_t>> moments() const {
            std::vector<std::tuple<Tensor, Tensor, int64_t>> out;
            for (const auto& p : params()) {
                auto it = optimizer_->state().find(p.unsafeGetTensorImpl());
                if (it == optimizer_->state().end()) {
                    out.emplace_back(Tensor(), Tensor(), 0);
                } else {
                    auto& s = static_cast<gs::training::FusedAdam::AdamParamState&>(*it->second);
                    out.emplace_back(s.exp_avg, s.exp_avg_sq, s.step_count);
                }
            }
            return out;
        }
        void zero_grad() { optimizer_->zero_grad(true, 0); }
        void set_active_sh_degree(int d) { sh_degree_ = d; }

    private:
        RefRender render(bool gut, const Tensor& viewmat, const Tensor& K, int width, int height, const Tensor& bg_color) {
            if (gut)
                return rasterize(viewmat, K, width, height, bg_color, 1.0f, false, 0, 0, std::nullopt, std::nullopt);
            auto Kc = K.cpu();
            auto a = Kc.accessor<float, 3>();
            return fast_rasterize(viewmat, a[0][0][0], a[0][1][1], a[0][0][2], a[0][1][2], width, height, bg_color);
        }

        Tensor means_, sh0_, shN_, scaling_, rotation_, opacity_, densification_info_;
        int sh_degree_;
        std::unique_ptr<gs::training::FusedAdam> optimizer_;
        std::unique_ptr<gs::training::ExponentialLR> scheduler_;
    };

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "The reference's own CUDA build of the training-step path (test infrastructure / timed comparator)";

    // ---- gsplat/Ops.h, one binding per operator (the same bindings the operator shim of this repository exposes)
#include "gsplat_ops_pybind.inc"

    // ---- loss, optimizer, regularizers, EWA rasterizer
    m.def("fusedssim", [](float C1, float C2, Tensor img1, Tensor img2, bool train) {
        return fusedssim(C1, C2, img1, img2, train);
    });
    m.def("fusedssim_backward", [](float C1, float C2, Tensor img1, Tensor img2, Tensor dL_dmap, Tensor dm_dmu1,
                                   Tensor dm_dsigma1_sq, Tensor dm_dsigma12) {
        return fusedssim_backward(C1, C2, img1, img2, dL_dmap, dm_dmu1, dm_dsigma1_sq, dm_dsigma12);
    });
    m.def("fused_ssim", [](Tensor img1, Tensor img2, std::string padding, bool train) {
        return fused_ssim(img1, img2, padding, train);
    });
    m.def("photometric_loss", &RefTrainer::photometric_loss);
    m.def("adam_step_wrapper", [](Tensor param, Tensor exp_avg, Tensor exp_avg_sq, Tensor param_grad, float lr, float beta1,
                                  float beta2, float eps, float bias_correction1, float bias_correction2_sqrt) {
        fast_gs::optimizer::adam_step_wrapper(param, exp_avg, exp_avg_sq, param_grad, lr, beta1, beta2, eps,
                                              bias_correction1, bias_correction2_sqrt);
    });
    m.def("exp_l1_regularization_with_grad", [](Tensor scaling_raw, float weight) {
        return gs::regularization::compute_exp_l1_regularization_with_grad_cuda(scaling_raw, weight);
    });
    m.def("sigmoid_l1_regularization_with_grad", [](Tensor opacity_raw, float weight) {
        return gs::regularization::compute_sigmoid_l1_regularization_with_grad_cuda(opacity_raw, weight);
    });
    m.def("fastgs_forward", [](Tensor means, Tensor scales_raw, Tensor rotations_raw, Tensor opacities_raw, Tensor sh0,
                               Tensor shN, Tensor w2c, Tensor cam_position, int active_sh_bases, int width, int height,
                               float fx, float fy, float cx, float cy, float near_plane, float far_plane) {
        return fast_gs::rasterization::forward_wrapper(means, scales_raw, rotations_raw, opacities_raw, sh0, shN, w2c,
                                                       cam_position, active_sh_bases, width, height, fx, fy, cx, cy,
                                                       near_plane, far_plane);
    });

    py::class_<RefRender>(m, "RefRender")
        .def_readonly("image", &RefRender::image)
        .def_readonly("alpha", &RefRender::alpha)
        .def_readonly("depth", &RefRender::depth)
        .def_readonly("radii", &RefRender::radii)
        .def_readonly("means2d", &RefRender::means2d)
        .def_readonly("depths", &RefRender::depths);

    py::class_<RefTrainer>(m, "RefTrainer")
        .def(py::init<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, std::vector<double>, int, int>())
        .def("rasterize", &RefTrainer::rasterize, py::call_guard<py::gil_scoped_release>())
        .def("fast_rasterize", &RefTrainer::fast_rasterize, py::call_guard<py::gil_scoped_release>())
        .def("render_no_grad", &RefTrainer::render_no_grad, py::call_guard<py::gil_scoped_release>())
        .def("forward_backward", &RefTrainer::forward_backward, py::call_guard<py::gil_scoped_release>())
        .def("train_step", &RefTrainer::train_step, py::call_guard<py::gil_scoped_release>())
        .def("optimizer_step", &RefTrainer::optimizer_step, py::call_guard<py::gil_scoped_release>())
        .def("params", &RefTrainer::params)
        .def("grads", &RefTrainer::grads)
        .def("moments", &RefTrainer::moments)
        .def("zero_grad", &RefTrainer::zero_grad)
        .def("set_active_sh_degree", &RefTrainer::set_active_sh_degree);
}
