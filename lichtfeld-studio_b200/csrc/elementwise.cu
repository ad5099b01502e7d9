// Streaming per-element / per-Gaussian kernels: fused Adam, operator-level SH, MCMC relocation,
// noise injection, quaternion -> matrix, and the index work of the MCMC densification step.
//
// Replaces src/training/fastgs/optimizer/include/adam_kernels.cuh:13 (K11, one launch for all six
// groups instead of six), gsplat/SphericalHarmonicsCUDA.cu:374 / :445 (K2 / K3), gsplat/RelocationCUDA.cu:12
// (K12) and :113 (K13), gsplat/QuatToRotmatCUDA.cu:13 (K14) and the ATen index glue of
// src/training/strategies/mcmc.cpp:112-347. All of it is HBM-bound.
#include "elementwise.cuh"
#include "gsmath.cuh"

namespace lfs {

namespace {

// ---- Adam -----------------------------------------------------------------------------------
__device__ __forceinline__ void adam_update(float& p, float& m, float& v, float g, float beta1, float beta2, float eps,
                                            float step_size, float bc2_sqrt_rcp) {
    const float m1 = beta1 * m + (1.0f - beta1) * g;
    const float m2 = beta2 * v + (1.0f - beta2) * g * g;
    const float denom = sqrtf(m2) * bc2_sqrt_rcp + eps;
    p -= step_size * m1 / denom;
    m = m1;
    v = m2;
}

__global__ void __launch_bounds__(256) adam_groups_kernel(AdamGroups G) {
    const int64_t total4 = G.prefix4[G.n_groups];
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total4; q += (int64_t)gridDim.x * blockDim.x) {
        int gi = 0;
#pragma unroll
        for (int k = 1; k < 6; ++k)
            if (k < G.n_groups && q >= G.prefix4[k]) gi = k;
        const AdamGroup& grp = G.g[gi];
        const int64_t e = (q - G.prefix4[gi]) * 4;
        if (grp.aligned && e + 4 <= grp.n) {
            float4 p = *reinterpret_cast<float4*>(grp.p + e);
            float4 m = *reinterpret_cast<float4*>(grp.m + e);
            float4 v = *reinterpret_cast<float4*>(grp.v + e);
            const float4 g = *reinterpret_cast<const float4*>(grp.g + e);
            adam_update(p.x, m.x, v.x, g.x * G.grad_scale, G.beta1, G.beta2, G.eps, grp.step_size, G.bc2_sqrt_rcp);
            adam_update(p.y, m.y, v.y, g.y * G.grad_scale, G.beta1, G.beta2, G.eps, grp.step_size, G.bc2_sqrt_rcp);
            adam_update(p.z, m.z, v.z, g.z * G.grad_scale, G.beta1, G.beta2, G.eps, grp.step_size, G.bc2_sqrt_rcp);
            adam_update(p.w, m.w, v.w, g.w * G.grad_scale, G.beta1, G.beta2, G.eps, grp.step_size, G.bc2_sqrt_rcp);
            *reinterpret_cast<float4*>(grp.p + e) = p;
            *reinterpret_cast<float4*>(grp.m + e) = m;
            *reinterpret_cast<float4*>(grp.v + e) = v;
        } else {
            for (int64_t i = e; i < e + 4 && i < grp.n; ++i) {
                float p = grp.p[i], m = grp.m[i], v = grp.v[i];
                adam_update(p, m, v, grp.g[i] * G.grad_scale, G.beta1, G.beta2, G.eps, grp.step_size, G.bc2_sqrt_rcp);
                grp.p[i] = p; grp.m[i] = m; grp.v[i] = v;
            }
        }
    }
}

__global__ void __launch_bounds__(256) adam_segments_kernel(AdamSegments S) {
    const int64_t total4 = S.prefix4[S.n];
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total4; q += (int64_t)gridDim.x * blockDim.x) {
        int gi = 0;
#pragma unroll
        for (int k = 1; k < kMaxAdamSegments; ++k)
            if (k < S.n && q >= S.prefix4[k]) gi = k;
        const AdamGroup& grp = S.g[gi];
        const int64_t e = (q - S.prefix4[gi]) * 4;
        if (grp.aligned && e + 4 <= grp.n) {
            float4 p = *reinterpret_cast<float4*>(grp.p + e);
            float4 m = *reinterpret_cast<float4*>(grp.m + e);
            float4 v = *reinterpret_cast<float4*>(grp.v + e);
            const float4 g = *reinterpret_cast<const float4*>(grp.g + e);
            adam_update(p.x, m.x, v.x, g.x * S.grad_scale, S.beta1, S.beta2, S.eps, grp.step_size, S.bc2_sqrt_rcp);
            adam_update(p.y, m.y, v.y, g.y * S.grad_scale, S.beta1, S.beta2, S.eps, grp.step_size, S.bc2_sqrt_rcp);
            adam_update(p.z, m.z, v.z, g.z * S.grad_scale, S.beta1, S.beta2, S.eps, grp.step_size, S.bc2_sqrt_rcp);
            adam_update(p.w, m.w, v.w, g.w * S.grad_scale, S.beta1, S.beta2, S.eps, grp.step_size, S.bc2_sqrt_rcp);
            *reinterpret_cast<float4*>(grp.p + e) = p;
            *reinterpret_cast<float4*>(grp.m + e) = m;
            *reinterpret_cast<float4*>(grp.v + e) = v;
        } else {
            for (int64_t i = e; i < e + 4 && i < grp.n; ++i) {
                float p = grp.p[i], m = grp.m[i], v = grp.v[i];
                adam_update(p, m, v, grp.g[i] * S.grad_scale, S.beta1, S.beta2, S.eps, grp.step_size, S.bc2_sqrt_rcp);
                grp.p[i] = p; grp.m[i] = m; grp.v[i] = v;
            }
        }
    }
}

// Reduce-scatter + Adam + all-gather in one pass over this rank's shard. Each element is summed by its
// owner only, in rank order, so every rank ends up with bit-identical parameters. Peer traffic is plain
// 16-byte loads over NVLink and, for the new parameters, either one plain 16-byte store per rank or one multimem.st
// through the NVSwitch multicast address of the buffer.
__global__ void __launch_bounds__(256) dp_reduce_adam_broadcast_kernel(DpArgs A) {
    const int64_t total4 = A.prefix4[A.n_segments];
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total4; q += (int64_t)gridDim.x * blockDim.x) {
        int si = 0;
#pragma unroll
        for (int k = 1; k < 6; ++k)
            if (k < A.n_segments && q >= A.prefix4[k]) si = k;
        const DpSegment& sg = A.seg[si];
        const int64_t e = (q - A.prefix4[si]) * 4;   // element within the segment (segments are 4-element aligned)
        const int64_t f = sg.offset + e;              // element within the flat buffers
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            if (r < A.world) {
                const float4 t = *reinterpret_cast<const float4*>(A.grads[r] + f);
                g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
            }
        }
        float4 p = *reinterpret_cast<const float4*>(A.params[0] + f);
        // every rank holds the same parameters; read the local copy (params[0] is this rank's own buffer)
        float4 m = *reinterpret_cast<float4*>(sg.m + e);
        float4 v = *reinterpret_cast<float4*>(sg.v + e);
        adam_update(p.x, m.x, v.x, g.x * A.grad_scale, A.beta1, A.beta2, A.eps, sg.step_size, A.bc2_sqrt_rcp);
        adam_update(p.y, m.y, v.y, g.y * A.grad_scale, A.beta1, A.beta2, A.eps, sg.step_size, A.bc2_sqrt_rcp);
        adam_update(p.z, m.z, v.z, g.z * A.grad_scale, A.beta1, A.beta2, A.eps, sg.step_size, A.bc2_sqrt_rcp);
        adam_update(p.w, m.w, v.w, g.w * A.grad_scale, A.beta1, A.beta2, A.eps, sg.step_size, A.bc2_sqrt_rcp);
        *reinterpret_cast<float4*>(sg.m + e) = m;
        *reinterpret_cast<float4*>(sg.v + e) = v;
        if (A.mc_params) {
            multimem_st4(A.mc_params + f, p);
        } else {
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < A.world) *reinterpret_cast<float4*>(A.params[r] + f) = p;
        }
    }
}

// ---- scale / opacity L1 regularisers --------------------------------------------------------------
__global__ void __launch_bounds__(256) regularization_kernel(int N, const float* __restrict__ scaling_raw,
                                                             const float* __restrict__ opacity_raw, float scale_gs,
                                                             float opac_gs, float* __restrict__ g_scaling,
                                                             float* __restrict__ g_opacity, float* __restrict__ loss) {
    __shared__ float red[2][8];
    float ssum = 0.f, osum = 0.f;
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < N; g += gridDim.x * blockDim.x) {
        if (scale_gs != 0.f) {
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float e = expf(scaling_raw[g * 3 + k]);
                ssum += e;
                g_scaling[g * 3 + k] += scale_gs * e;
            }
        }
        if (opac_gs != 0.f) {
            const float s = 1.0f / (1.0f + expf(-opacity_raw[g]));
            osum += s;
            g_opacity[g] += opac_gs * s * (1.0f - s);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
        osum += __shfl_xor_sync(0xffffffffu, osum, o);
    }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ssum; red[1][threadIdx.x >> 5] = osum; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f, b = 0.f;
        for (int k = 0; k < 8; ++k) { a += red[0][k]; b += red[1][k]; }
        // grad scale = weight / n, so weight * mean = grad scale * sum
        if (scale_gs != 0.f) atomicAdd(&loss[0], a * scale_gs);
        if (opac_gs != 0.f) atomicAdd(&loss[1], b * opac_gs);
    }
}

// ---- spherical harmonics, operator level ------------------------------------------------------
__global__ void __launch_bounds__(256) sh_fwd_kernel(int n, int K, int degree, const float* __restrict__ dirs,
                                                     const float* __restrict__ coeffs, const uint8_t* __restrict__ masks,
                                                     float* __restrict__ colors) {
    const int nb = (degree + 1) * (degree + 1);
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n; e += gridDim.x * blockDim.x) {
        if (masks && !masks[e]) continue;
        float B[25];
        sh_basis(degree, dirs[e * 3], dirs[e * 3 + 1], dirs[e * 3 + 2], B);
        const float* cf = coeffs + (size_t)e * K * 3;
        float r = 0.f, g = 0.f, b = 0.f;
        for (int k = 0; k < nb; ++k) { r += B[k] * cf[k * 3]; g += B[k] * cf[k * 3 + 1]; b += B[k] * cf[k * 3 + 2]; }
        colors[e * 3] = r; colors[e * 3 + 1] = g; colors[e * 3 + 2] = b;
    }
}

__global__ void __launch_bounds__(256) sh_bwd_kernel(int n, int K, int degree, const float* __restrict__ dirs,
                                                     const uint8_t* __restrict__ masks, const float* __restrict__ v_colors,
                                                     float* __restrict__ v_coeffs) {
    const int nb = (degree + 1) * (degree + 1);
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n; e += gridDim.x * blockDim.x) {
        float* vc = v_coeffs + (size_t)e * K * 3;
        if (masks && !masks[e]) {
            for (int k = 0; k < K * 3; ++k) vc[k] = 0.f;
            continue;
        }
        float B[25];
        sh_basis(degree, dirs[e * 3], dirs[e * 3 + 1], dirs[e * 3 + 2], B);
        const float r = v_colors[e * 3], g = v_colors[e * 3 + 1], b = v_colors[e * 3 + 2];
        for (int k = 0; k < K; ++k) {
            const float w = k < nb ? B[k] : 0.f;
            vc[k * 3] = w * r; vc[k * 3 + 1] = w * g; vc[k * 3 + 2] = w * b;
        }
    }
}

// ---- MCMC ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) relocation_kernel(int n, const float* __restrict__ opacities, const float* __restrict__ scales,
                                                         const int32_t* __restrict__ ratios, const float* __restrict__ binoms,
                                                         int n_max, float* __restrict__ new_opacities, float* __restrict__ new_scales) {
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
        const int n_idx = ratios[idx];
        const float op = opacities[idx];
        const float no = 1.0f - powf(1.0f - op, 1.0f / (float)n_idx);
        new_opacities[idx] = no;
        // denom = sum_{i=1..n} sum_{k<i} C(i-1,k) (-1)^k no^(k+1) / sqrt(k+1), same summation order
        float denom_sum = 0.0f;
        for (int i = 1; i <= n_idx; ++i) {
            float pw = no;  // no^(k+1)
            for (int k = 0; k <= i - 1; ++k) {
                const float sign = (k & 1) ? -1.0f : 1.0f;
                const float term = (sign / sqrtf((float)(k + 1))) * pw;
                denom_sum += binoms[(i - 1) * n_max + k] * term;
                pw *= no;
            }
        }
        const float coeff = op / denom_sum;
#pragma unroll
        for (int k = 0; k < 3; ++k) new_scales[idx * 3 + k] = coeff * scales[idx * 3 + k];
    }
}

__global__ void __launch_bounds__(256) add_noise_kernel(int n, const float* __restrict__ raw_opacities, const float* __restrict__ raw_scales,
                                                        const float* __restrict__ raw_quats, const float* __restrict__ noise,
                                                        float* __restrict__ means, float current_lr) {
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
        const float s2[3] = {__expf(2.f * raw_scales[idx * 3]), __expf(2.f * raw_scales[idx * 3 + 1]), __expf(2.f * raw_scales[idx * 3 + 2])};
        const float4 q = reinterpret_cast<const float4*>(raw_quats)[idx];
        float w = q.x, x = q.y, y = q.z, z = q.w;
        const float inv_norm = fminf(rsqrtf(x * x + y * y + z * z + w * w), 1e+12f);
        x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
        const float x2 = x * x, y2 = y * y, z2 = z * z, xy = x * y, xz = x * z, yz = y * z, wx = w * x, wy = w * y, wz = w * z;
        const float R[9] = {1.f - 2.f * (y2 + z2), 2.f * (xy - wz), 2.f * (xz + wy),
                            2.f * (xy + wz), 1.f - 2.f * (x2 + z2), 2.f * (yz - wx),
                            2.f * (xz - wy), 2.f * (yz + wx), 1.f - 2.f * (x2 + y2)};
        const float nz[3] = {noise[idx * 3], noise[idx * 3 + 1], noise[idx * 3 + 2]};
        // (R S^2 R^T) noise = R (S^2 (R^T noise))
        float tmp[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) tmp[k] = s2[k] * (R[0 * 3 + k] * nz[0] + R[1 * 3 + k] * nz[1] + R[2 * 3 + k] * nz[2]);
        const float opacity = 1.0f / (1.f + __expf(-raw_opacities[idx]));
        const float op_sigmoid = 1.0f / (1.f + __expf(100.f * opacity - 0.5f));
        const float nf = current_lr * op_sigmoid;
#pragma unroll
        for (int a = 0; a < 3; ++a)
            means[idx * 3 + a] += nf * (R[a * 3 + 0] * tmp[0] + R[a * 3 + 1] * tmp[1] + R[a * 3 + 2] * tmp[2]);
    }
}

__global__ void __launch_bounds__(256) quats_to_rotmats_kernel(int n, const float* __restrict__ quats, float* __restrict__ rotmats) {
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
        const float4 q = reinterpret_cast<const float4*>(quats)[idx];
        float R[9], inv_norm, qn[4];
        quat_to_rotmat_renorm(q.x, q.y, q.z, q.w, R, inv_norm, qn);
#pragma unroll
        for (int k = 0; k < 9; ++k) rotmats[(size_t)idx * 9 + k] = R[k];
    }
}

// float32 sigmoid / exp exactly as ATen evaluates them (1 / (1 + exp(-x)) in float): the MCMC sampling
// probabilities and the dead mask must be the values torch::sigmoid gives, or multinomial draws differ.
__device__ __forceinline__ float sigmoid_d(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(256) mcmc_flags_kernel(int N, const float* __restrict__ opacity_raw, const float* __restrict__ rotation_raw,
                                                         float min_opacity, int32_t* __restrict__ flags) {
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < N; g += gridDim.x * blockDim.x) {
        const float4 q = reinterpret_cast<const float4*>(rotation_raw)[g];
        const float n2 = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
        flags[g] = (sigmoid_d(opacity_raw[g]) <= min_opacity || n2 < 1e-8f) ? 1 : 0;
    }
}

__global__ void __launch_bounds__(256) mcmc_compact_kernel(int N, const int32_t* __restrict__ flags, const int32_t* __restrict__ dead_offs,
                                                           const int32_t* __restrict__ n_dead_dev, const float* __restrict__ opacity_raw,
                                                           int64_t* __restrict__ dead_indices, int64_t* __restrict__ alive_indices,
                                                           float* __restrict__ alive_opacities, int32_t* __restrict__ counts) {
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < N; g += gridDim.x * blockDim.x) {
        const int d = dead_offs[g];
        if (flags[g]) {
            dead_indices[d] = g;
        } else {
            const int a = g - d;
            alive_indices[a] = g;
            alive_opacities[a] = sigmoid_d(opacity_raw[g]);
        }
        if (g == 0) { counts[0] = *n_dead_dev; counts[1] = N - *n_dead_dev; }
    }
}

__global__ void __launch_bounds__(256) mcmc_map_indices_kernel(int n, const int64_t* __restrict__ local, const int64_t* __restrict__ map,
                                                               int64_t* __restrict__ out) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = map[local[i]];
}

__global__ void __launch_bounds__(256) mcmc_count_kernel(int n, const int64_t* __restrict__ sampled, int32_t* __restrict__ counts) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) atomicAdd(&counts[sampled[i]], 1);
}

__global__ void __launch_bounds__(256) mcmc_gather_kernel(int n, const int64_t* __restrict__ sampled, const int32_t* __restrict__ counts,
                                                          const float* __restrict__ opacity_raw, const float* __restrict__ scaling_raw,
                                                          int n_max, int32_t* __restrict__ ratios, float* __restrict__ s_opac,
                                                          float* __restrict__ s_scales) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int64_t g = sampled[i];
        ratios[i] = max(1, min(1 + counts[g], n_max));
        s_opac[i] = sigmoid_d(opacity_raw[g]);
#pragma unroll
        for (int k = 0; k < 3; ++k) s_scales[i * 3 + k] = expf(scaling_raw[g * 3 + k]);
    }
}

__global__ void __launch_bounds__(256) mcmc_writeback_kernel(int n, const int64_t* __restrict__ sampled, const float* __restrict__ new_opac,
                                                             const float* __restrict__ new_scales, float min_opacity,
                                                             float* __restrict__ opacity_raw, float* __restrict__ scaling_raw) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int64_t g = sampled[i];
        const float o = fminf(fmaxf(new_opac[i], min_opacity), 1.0f - 1e-7f);
        opacity_raw[g] = logf(o / (1.0f - o));
#pragma unroll
        for (int k = 0; k < 3; ++k) scaling_raw[g * 3 + k] = logf(new_scales[i * 3 + k]);
    }
}

struct RowTable {
    float* p[6]; float* m[6]; float* v[6];
    int width[6];
    int prefix[7];
};

// Copies the 6 parameter rows src -> dst and zeroes the moments: at the source rows when relocating
// (zero_at_dst == 0), at the destination rows when appending.
__global__ void __launch_bounds__(256) mcmc_copy_rows_kernel(int n, int64_t N, const int64_t* __restrict__ sampled,
                                                             const int64_t* __restrict__ dst_indices, RowTable T, int zero_at_dst) {
    const int row_w = T.prefix[6];
    const int64_t total = (int64_t)n * row_w;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(q / row_w), j = (int)(q % row_w);
        int gi = 0;
#pragma unroll
        for (int k = 1; k < 6; ++k)
            if (j >= T.prefix[k]) gi = k;
        const int col = j - T.prefix[gi], w = T.width[gi];
        const int64_t src = sampled[i];
        const int64_t dst = dst_indices ? dst_indices[i] : (N + i);
        T.p[gi][dst * w + col] = T.p[gi][src * w + col];
        const int64_t z = zero_at_dst ? dst : src;
        if (T.m[gi]) T.m[gi][z * w + col] = 0.f;
        if (T.v[gi]) T.v[gi][z * w + col] = 0.f;
    }
}

}  // namespace

int launch_adam_groups(const AdamGroups& G, cudaStream_t st) {
    const int64_t total4 = G.prefix4[G.n_groups];
    if (total4 == 0) return LFS_OK;
    LFS_TIMED("adam", st);
    adam_groups_kernel<<<grid_for(total4, 256, 16), 256, 0, st>>>(G);
    return check_launch("adam_groups");
}

int launch_adam_segments(const AdamSegments& S, int ctas_per_sm, cudaStream_t st) {
    const int64_t total4 = S.prefix4[S.n];
    if (total4 == 0) return LFS_OK;
    LFS_TIMED("adam", st);
    adam_segments_kernel<<<grid_for(total4, 256, ctas_per_sm > 0 ? ctas_per_sm : 16), 256, 0, st>>>(S);
    return check_launch("adam_segments");
}

int launch_dp_reduce_adam_broadcast(const DpArgs& A, int ctas_per_sm, cudaStream_t st) {
    const int64_t total4 = A.prefix4[A.n_segments];
    if (total4 == 0) return LFS_OK;
    // two names so that a profile tells the exchange on the caller's stream from the small-footprint launch that
    // overlaps the next step's kernels on a side stream
    LFS_TIMED(ctas_per_sm > 0 ? "dp_exchange_side" : "dp_exchange_main", st);
    // NVLink-bound: a few CTAs per SM keep enough 16-byte requests in flight; a caller that runs other kernels
    // next to this one asks for a small footprint so that those kernels find free thread slots
    dp_reduce_adam_broadcast_kernel<<<grid_for(total4, 256, ctas_per_sm > 0 ? ctas_per_sm : 16), 256, 0, st>>>(A);
    return check_launch("dp_reduce_adam_broadcast");
}

// ---------------------------------------------------------------------------------------------
// Cross-GPU ordering by flags in peer-mapped memory (no counterpart in the reference, which is single-GPU).
// dp_signal_kernel runs after a producer kernel on the same stream and stores a step number into one word of every
// peer's flag array; dp_wait_kernel spins until the words written by all ranks have reached a step number, for at most
// timeout_ns (globaltimer). On expiry it records which ranks were missing and RETURNS: the stream goes on, nothing
// hangs, and the host reads the status word to learn that a rank stopped stepping.
// ---------------------------------------------------------------------------------------------
struct DpPeers { int32_t* flags[LFS_DP_MAX_WORLD]; };

__global__ void dp_signal_kernel(DpPeers peers, int world, int own_rank, int slot, int32_t value) {
    const int r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();   // this stream's earlier writes (also to peer memory) are ordered before the flag
    int32_t* dst = peers.flags[r] + slot * LFS_DP_MAX_WORLD + own_rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(value) : "memory");
}

// Lane r waits until rank r's word of `slot` shows `value` or a later step, for at most timeout_ns of the global timer. A
// wait that runs out records itself in status[0..3] = {1, bit mask of the missing ranks, slot, value of the FIRST failed
// wait} and returns like a satisfied one: nothing ever spins without a limit, and the host learns of it from the status.
__device__ __forceinline__ void dp_wait_lane(const int32_t* __restrict__ flags, int world, int slot, int32_t value,
                                             unsigned long long timeout_ns, int32_t* __restrict__ status) {
    const int r = threadIdx.x;
    if (r < world) {
        const int32_t* src = flags + slot * LFS_DP_MAX_WORLD + r;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        bool ok = false;
        for (;;) {
            int32_t seen;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(src) : "memory");
            if (seen - value >= 0) { ok = true; break; }          // step numbers only grow (wrap-safe comparison)
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > timeout_ns) break;
            __nanosleep(100);
        }
        if (!ok) {
            atomicOr(&status[1], 1 << r);         // ranks that were missing
            if (atomicOr(&status[0], 1) == 0) {   // a wait ran out; the first one names slot and step
                status[2] = slot;
                status[3] = value;
            }
        }
    }
    __syncwarp();
    __threadfence_system();   // data written before the flags is visible to the kernels that follow on this stream
}

__global__ void dp_wait_kernel(const int32_t* __restrict__ flags, int world, int slot, int32_t value, unsigned long long timeout_ns,
                               int32_t* __restrict__ status) {
    dp_wait_lane(flags, world, slot, value, timeout_ns, status);
}

// signal + wait in one launch: the rendezvous of the data-parallel step
__global__ void dp_barrier_kernel(DpPeers peers, int world, int own_rank, int slot, int32_t value, unsigned long long timeout_ns,
                                  int32_t* __restrict__ status) {
    const int r = threadIdx.x;
    if (r < world) {
        __threadfence_system();
        int32_t* dst = peers.flags[r] + slot * LFS_DP_MAX_WORLD + own_rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(value) : "memory");
    }
    dp_wait_lane(peers.flags[own_rank], world, slot, value, timeout_ns, status);
}

int launch_dp_signal(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, cudaStream_t st) {
    DpPeers p;
    for (int i = 0; i < LFS_DP_MAX_WORLD; ++i) p.flags[i] = i < world ? peer_flags[i] : nullptr;
    dp_signal_kernel<<<1, 32, 0, st>>>(p, world, own_rank, slot, value);
    return check_launch("dp_signal");
}

int launch_dp_wait(int world, const int32_t* flags, int slot, int32_t value, uint64_t timeout_ns, int32_t* status, cudaStream_t st) {
    dp_wait_kernel<<<1, 32, 0, st>>>(flags, world, slot, value, (unsigned long long)timeout_ns, status);
    return check_launch("dp_wait");
}

int launch_dp_barrier(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, uint64_t timeout_ns, int32_t* status,
                      cudaStream_t st) {
    DpPeers p;
    for (int i = 0; i < LFS_DP_MAX_WORLD; ++i) p.flags[i] = i < world ? peer_flags[i] : nullptr;
    dp_barrier_kernel<<<1, 32, 0, st>>>(p, world, own_rank, slot, value, (unsigned long long)timeout_ns, status);
    return check_launch("dp_barrier");
}

int launch_regularization(int N, const float* scaling_raw, const float* opacity_raw, float scale_weight, float opacity_weight,
                          float* g_scaling, float* g_opacity, float* loss, cudaStream_t st) {
    cudaMemsetAsync(loss, 0, 2 * sizeof(float), st);
    if (N == 0) return LFS_OK;
    LFS_TIMED("regularization", st);
    regularization_kernel<<<grid_for(N, 256, 4), 256, 0, st>>>(N, scaling_raw, opacity_raw, scale_weight / (3.0f * (float)N),
                                                               opacity_weight / (float)N, g_scaling, g_opacity, loss);
    return check_launch("regularization");
}

int launch_sh_fwd(int n, int K, int degree, const float* dirs, const float* coeffs, const uint8_t* masks, float* colors, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    sh_fwd_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, K, degree, dirs, coeffs, masks, colors);
    return check_launch("sh_fwd");
}
int launch_sh_bwd(int n, int K, int degree, const float* dirs, const uint8_t* masks, const float* v_colors, float* v_coeffs, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    sh_bwd_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, K, degree, dirs, masks, v_colors, v_coeffs);
    return check_launch("sh_bwd");
}
int launch_relocation(int n, const float* opacities, const float* scales, const int32_t* ratios, const float* binoms, int n_max,
                      float* new_opacities, float* new_scales, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    relocation_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, opacities, scales, ratios, binoms, n_max, new_opacities, new_scales);
    return check_launch("relocation");
}
int launch_add_noise(int n, const float* raw_opacities, const float* raw_scales, const float* raw_quats, const float* noise,
                     float* means, float lr, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    add_noise_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, raw_opacities, raw_scales, raw_quats, noise, means, lr);
    return check_launch("add_noise");
}
int launch_quats_to_rotmats(int n, const float* quats, float* rotmats, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    quats_to_rotmats_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, quats, rotmats);
    return check_launch("quats_to_rotmats");
}

// ---------------------------------------------------------------------------------------------
// PLY vertex rows (src/core/splat_data.cpp:402-418 attribute order, :483-503 contents):
//   x y z | nx ny nz (zeros) | f_dc_0..2 | f_rest_* channel-major (transpose(1,2).flatten(1)) |
//   opacity (raw logit) | scale_0..2 (raw log) | rot_0..3 (F.normalize: q / max(|q|, 1e-12))
// One warp per row: lanes stride over the row's 14 + 3 K floats, so both the reads of the six tensors
// and the interleaved row writes are contiguous runs. Explicit _rn arithmetic: the norm does not
// depend on the compiler's FMA contraction.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ply_rows_pack_kernel(int N, int K, lfs_splats p, float* __restrict__ rows) {
    const int width = 14 + 3 * K, rest = K - 1;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < N; g += warps) {
        float* row = rows + (size_t)g * width;
        const float4 q = reinterpret_cast<const float4*>(p.rotation_raw)[g];
        const float n2 = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(q.x, q.x), __fmul_rn(q.y, q.y)), __fmul_rn(q.z, q.z)), __fmul_rn(q.w, q.w));
        const float nrm = fmaxf(__fsqrt_rn(n2), 1e-12f);
        for (int c = lane; c < width; c += 32) {
            float v;
            if (c < 3) v = p.means[g * 3 + c];
            else if (c < 6) v = 0.f;
            else if (c < 9) v = p.sh0[g * 3 + (c - 6)];
            else if (c < 9 + 3 * rest) { const int i = c - 9, ch = i / rest, k = i % rest; v = p.shN[((size_t)g * rest + k) * 3 + ch]; }
            else if (c == 9 + 3 * rest) v = p.opacity_raw[g];
            else if (c < 13 + 3 * rest) v = p.scaling_raw[g * 3 + (c - 10 - 3 * rest)];
            else { const int k = c - 13 - 3 * rest; v = __fdiv_rn(k == 0 ? q.x : k == 1 ? q.y : k == 2 ? q.z : q.w, nrm); }
            row[c] = v;
        }
    }
}

// Inverse of ply_rows_pack_kernel (normals are ignored; the quaternion is stored as it is in the file).
__global__ void __launch_bounds__(256) ply_rows_unpack_kernel(int N, int K, const float* __restrict__ rows, lfs_splats p) {
    const int width = 14 + 3 * K, rest = K - 1;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < N; g += warps) {
        const float* row = rows + (size_t)g * width;
        for (int c = lane; c < width; c += 32) {
            const float v = row[c];
            if (c < 3) p.means[g * 3 + c] = v;
            else if (c < 6) {}
            else if (c < 9) p.sh0[g * 3 + (c - 6)] = v;
            else if (c < 9 + 3 * rest) { const int i = c - 9, ch = i / rest, k = i % rest; p.shN[((size_t)g * rest + k) * 3 + ch] = v; }
            else if (c == 9 + 3 * rest) p.opacity_raw[g] = v;
            else if (c < 13 + 3 * rest) p.scaling_raw[g * 3 + (c - 10 - 3 * rest)] = v;
            else p.rotation_raw[g * 4 + (c - 13 - 3 * rest)] = v;
        }
    }
}

int launch_ply_rows(int N, int K, const lfs_splats& p, float* rows, int unpack, cudaStream_t st) {
    if (N == 0) return LFS_OK;
    LFS_TIMED(unpack ? "ply_rows_unpack" : "ply_rows_pack", st);
    const int grid = (int)min((int64_t)num_sms() * 8, ((int64_t)N * 32 + 255) / 256);
    if (unpack) ply_rows_unpack_kernel<<<grid, 256, 0, st>>>(N, K, rows, p);
    else ply_rows_pack_kernel<<<grid, 256, 0, st>>>(N, K, p, rows);
    return check_launch("ply_rows");
}

int launch_mcmc_classify(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity, int64_t* dead_indices,
                         int64_t* alive_indices, float* alive_opacities, int32_t* counts_dev, int32_t* flags, int32_t* offs,
                         int32_t* total_dev, const SortScratch& s, cudaStream_t st) {
    if (N == 0) { cudaMemsetAsync(counts_dev, 0, 2 * sizeof(int32_t), st); return LFS_OK; }
    mcmc_flags_kernel<<<grid_for(N, 256), 256, 0, st>>>(N, opacity_raw, rotation_raw, min_opacity, flags);
    const int rc = exclusive_scan_gather(flags, nullptr, N, offs, total_dev, s, st);
    if (rc != LFS_OK) return rc;
    mcmc_compact_kernel<<<grid_for(N, 256), 256, 0, st>>>(N, flags, offs, total_dev, opacity_raw, dead_indices, alive_indices,
                                                          alive_opacities, counts_dev);
    return check_launch("mcmc_classify");
}

int launch_mcmc_map_indices(int n, const int64_t* local, const int64_t* map, int64_t* out, cudaStream_t st) {
    if (n == 0) return LFS_OK;
    mcmc_map_indices_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, local, map, out);
    return check_launch("mcmc_map_indices");
}

int launch_mcmc_gather_ratios(int N, int n, const int64_t* sampled, const float* opacity_raw, const float* scaling_raw, int n_max,
                              int32_t* counts, int32_t* ratios, float* s_opac, float* s_scales, cudaStream_t st) {
    cudaMemsetAsync(counts, 0, (size_t)N * sizeof(int32_t), st);
    if (n == 0) return LFS_OK;
    mcmc_count_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, sampled, counts);
    mcmc_gather_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, sampled, counts, opacity_raw, scaling_raw, n_max, ratios, s_opac, s_scales);
    return check_launch("mcmc_gather_ratios");
}

int launch_mcmc_apply(int N, int K, int n, const int64_t* sampled, const int64_t* dst_indices, const float* new_opac,
                      const float* new_scales, float min_opacity, const lfs_splats& p, const lfs_splats* m, const lfs_splats* v,
                      cudaStream_t st) {
    if (n == 0) return LFS_OK;
    mcmc_writeback_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, sampled, new_opac, new_scales, min_opacity, p.opacity_raw, p.scaling_raw);
    RowTable T;
    float* pp[6] = {p.means, p.sh0, p.shN, p.scaling_raw, p.rotation_raw, p.opacity_raw};
    const int w[6] = {3, 3, (K - 1) * 3, 3, 4, 1};
    T.prefix[0] = 0;
    for (int k = 0; k < 6; ++k) {
        T.p[k] = pp[k];
        T.width[k] = w[k];
        T.prefix[k + 1] = T.prefix[k] + w[k];
        T.m[k] = nullptr; T.v[k] = nullptr;
    }
    if (m) { float* a[6] = {m->means, m->sh0, m->shN, m->scaling_raw, m->rotation_raw, m->opacity_raw}; for (int k = 0; k < 6; ++k) T.m[k] = a[k]; }
    if (v) { float* a[6] = {v->means, v->sh0, v->shN, v->scaling_raw, v->rotation_raw, v->opacity_raw}; for (int k = 0; k < 6; ++k) T.v[k] = a[k]; }
    const int64_t total = (int64_t)n * T.prefix[6];
    mcmc_copy_rows_kernel<<<grid_for(total, 256), 256, 0, st>>>(n, (int64_t)N, sampled, dst_indices, T, dst_indices ? 0 : 1);
    return check_launch("mcmc_apply");
}

}  // namespace lfs
