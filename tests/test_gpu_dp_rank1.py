"""The data-parallel rank-1 shN update (lfs_dp_sh_rank1_adam_broadcast) on ONE GPU: the "ranks" are cameras whose
factor buffers and parameter copies live on the same device (2, 4 and 8 of them), so the kernel's peer pointers are plain local pointers.
Reference: the materialised gradients of both cameras accumulated, then lfs_adam_step_splats."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("n,deg,world,active,pad", [(6000, 3, 2, 3, 0), (4004, 2, 2, 2, 0), (6000, 3, 4, 3, 0), (5000, 3, 8, 3, 0),
                                                      (5001, 3, 2, 2, 59)])   # active degree below the stored one, padded capacity
def test_emulated_ranks_equal_accumulated_gradients(pkg, synth, n, deg, world, active, pad):
    tr, capi = pkg.trainer, pkg._capi
    W, H, K = 160, 120, (deg + 1) ** 2
    rest = (K - 1) * 3
    cfg, P, vm0, Kmat = make_scene(synth, n, W, H, deg, seed=31)
    poses = synth.hemisphere_poses(8, 4.0)
    cams = [tr.Camera(T(vm0), T(Kmat), W, H)] + [tr.Camera(T(poses[(3 * r) % 8]), T(Kmat), W, H) for r in range(1, world)]
    bg = T(np.array([0.1, 0.4, 0.2], np.float32))
    rng = np.random.default_rng(2)
    vr = [T(rng.normal(size=(H, W, 3)).astype(np.float32)) for _ in range(world)]

    def fresh():
        model = tr.SplatData(n, K, DEV, n + pad).load(P)
        m, v = model.like(), model.like()
        gen = torch.Generator(device=DEV).manual_seed(5)
        m.flat.copy_(torch.randn(m.flat.shape, generator=gen, device=DEV) * 1e-3)
        v.flat.copy_(torch.rand(v.flat.shape, generator=gen, device=DEV) * 1e-4 + 1e-6)
        return model, m, v

    # reference: accumulate both cameras' materialised gradients, one Adam step with the mean
    ref, m_ref, v_ref = fresh()
    rast = tr.Rasterizer(ref, W, H, active)
    grads = ref.like()
    for r in range(world):
        rast.forward(cams[r], bg)
        rast.backward(vr[r], grads, bg, accumulate=(r > 0))
    tr.adam_step_splats(ref, m_ref, v_ref, grads, LRS, 2, grad_scale=1.0 / world)

    # emulated ranks: each camera's factors, then the kernel with two "peers"
    copies = [fresh() for _ in range(world)]
    facs = []
    for r in range(world):
        model = copies[r][0]
        rr = tr.Rasterizer(model, W, H, active)
        g = model.like()
        rr.forward(cams[r], bg)
        rr.backward(vr[r], g, bg, sh_factors=True)
        facs.append(g)
    _, m_own, v_own = copies[0]
    total = copies[0][0].capacity * rest          # the whole tensor, rows beyond n included (zero gradient there)
    cut = (total // 2) // 4 * 4 + 4          # a 4-aligned cut inside a row
    assert cut % rest != 0
    stream = capi.vp(torch.cuda.current_stream().cuda_stream)
    pf = (C.c_void_p * world)(*[facs[r].tensor("shN").data_ptr() for r in range(world)])
    ps = (C.c_void_p * world)(*[copies[r][0].tensor("shN").data_ptr() for r in range(world)])
    for lo, cnt in ((0, cut), (cut, total - cut)):
        capi.call("lfs_dp_sh_rank1_adam_broadcast", world, pf, ps, None, n, K, active, lo, cnt,
                  capi.vp(m_own.tensor("shN").data_ptr() + 4 * lo), capi.vp(v_own.tensor("shN").data_ptr() + 4 * lo),
                  LRS[2], 0.9, 0.999, 1e-15, 2, 1.0 / world, 0, stream)
    torch.cuda.synchronize()
    a = copies[0][0].tensor("shN")
    for r in range(1, world):
        assert torch.equal(a, copies[r][0].tensor("shN"))      # every "rank" received the same coefficients
    p0 = T(P["shN"]).reshape(a.shape)
    assert rel_l2((a - p0).cpu().numpy(), (ref.tensor("shN") - p0).cpu().numpy()) < 1e-3
    assert rel_l2(m_own.tensor("shN").cpu().numpy(), m_ref.tensor("shN").cpu().numpy()) < 1e-5
    assert rel_l2(v_own.tensor("shN").cpu().numpy(), v_ref.tensor("shN").cpu().numpy()) < 1e-5
    # the factor rows: zero colour gradient exactly where the Gaussian was not visible, unit directions elsewhere
    f = facs[0].tensor("shN").reshape(-1)[: n * 6].reshape(n, 6)
    nz = f[:, :3].abs().sum(1) > 0
    assert bool(nz.any()) and float((f[nz, 3:].norm(dim=1) - 1).abs().max()) < 1e-5


def test_factors_cannot_be_accumulated(pkg, synth):
    tr, capi = pkg.trainer, pkg._capi
    n, W, H, deg = 2000, 64, 48, 1
    cfg, P, vm, Kmat = make_scene(synth, n, W, H, deg, seed=4)
    model = tr.SplatData(n, 4, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg)
    rast.forward(tr.Camera(T(vm), T(Kmat), W, H), None)
    v = torch.zeros(H, W, 3, device=DEV)
    with pytest.raises(capi.LfsError):
        rast.backward(v, model.like(), None, accumulate=True, sh_factors=True)
