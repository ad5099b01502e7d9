// Python module around the operator shim (ops_shim.cpp): the twelve operators of gsplat/Ops.h with the reference's
// signatures, served by the lfs_b200 C ABI. Used by the drop-in test, which drives this module and the reference's own
// build through the same call sequence, and usable from Python wherever torch tensors are at hand.
#include <torch/extension.h>

#include <optional>
#include <vector>

#include "lfs_gsplat_ops.h"

namespace {
    using torch::Tensor;
    using OptTensor = std::optional<Tensor>;

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
} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "namespace gsplat of gsplat/Ops.h on the lfs_b200 C ABI";
#include "gsplat_ops_pybind.inc"
}
