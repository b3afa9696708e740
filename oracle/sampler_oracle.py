"""CPU oracle for K-Fold's sampler loop (ECSI bridge sampler).  TEST INFRASTRUCTURE ONLY.

Restates, in plain PyTorch, what ``KFoldECSI.sample_structure`` (model/modules/ecsi.py:468-560) does around the score
network: random augmentation, forward-pinned churn, bridge preconditioning, rotation-only rigid alignment, centring and
the SI / ECSI update.  Nothing under ``kfold_b200/`` may import this file.

Every random draw goes through a ``rng`` object with one method, ``randn(shape) -> float32 CPU tensor``; the draws happen
in the reference's order (rotation quaternions, translation, churn noise, update noise), so a tape of pre-generated
normals reproduces a reference run that consumed the same tape.  Parity is pinned by ``tests/golden/sampler_*.npz``,
produced by the real ``KFoldECSI`` class with ``torch.randn`` / ``torch.randn_like`` reading from such a tape.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import pairformer_oracle as O


class NoiseTape:
    """Standard normals from ``numpy.random.RandomState(seed)`` in call order (frozen across numpy versions)."""

    def __init__(self, seed: int):
        self.rs = np.random.RandomState(seed)
        self.calls = 0

    def randn(self, shape) -> torch.Tensor:
        self.calls += 1
        return torch.from_numpy(self.rs.standard_normal(tuple(shape)).astype(np.float32))


# ----------------------------------------------------------------------------- coefficients (ecsi.py:106-131, :373-417)
def _clip(t: float, eps: float = 1e-10) -> float:
    return max(t, eps)


def _sqrt(t: float) -> float:
    return max(t, 0.0) ** 0.5


class Coeffs:
    """SICoeffs (ecsi.py:106-131): alpha = 1 - t, beta = t, gamma = 2 gamma_max sqrt(t (1 - t))."""

    def __init__(self, gamma_max: float):
        self.gamma_max = gamma_max

    def alpha(self, t): return 1.0 - t
    def beta(self, t): return t
    def gamma(self, t): return 2 * self.gamma_max * _sqrt(t * (1 - t))
    def gamma_deriv(self, t): return self.gamma_max * (1 - 2 * t) / _clip(_sqrt(t * (1 - t)))
    def sigma_eff(self, t): return self.gamma(t) / _clip(self.alpha(t))


DEFAULTS = dict(sigma_0=16.0, sigma_T=27.0, cov_0T=175.0, time_min=1e-8, time_max=0.9999, gamma_max=6.0,
                time_schedule_boundary=0.5, sample_step_fraction=(0.4, 0.6), sample_time_power=(0.5, 2.0),
                sde_end_time=0.1, eta=1.0, step_scale=1.0, churn_end_time=0.5, churn_factor_range=(0.1, 0.4))


def bridge_scalings(cfg: dict, t: float):
    """``_get_bridge_scalings`` (ecsi.py:373-417) for a float time."""
    C = Coeffs(cfg["gamma_max"])
    a, b, g = C.alpha(t), C.beta(t), C.gamma(t)
    s0, sT, cov = cfg["sigma_0"], cfg["sigma_T"], cfg["cov_0T"]
    c_in = 1 / _clip(_sqrt((a * s0) ** 2 + (b * sT) ** 2 + 2 * a * b * cov + g ** 2))
    c_skip = (a * s0 ** 2 + b * cov) * (c_in ** 2)
    c_out = _sqrt((b * s0 * sT) ** 2 - (b * cov) ** 2 + g ** 2 * s0 ** 2) * c_in
    return c_in, c_skip, c_out


def c_noise(t: float) -> float:
    """ecsi.py:431-433."""
    return 0.25 * math.log(_clip(t, 1e-10))


def sampling_schedule(cfg: dict, num_steps: int) -> list:
    """``get_sampling_schedule`` (ecsi.py:438-466): two power-law intervals joined at the boundary, then zero."""
    progress = np.linspace(0.0, 1.0, num_steps)
    high_steps, low_steps = cfg["sample_step_fraction"]
    high_power, low_power = cfg["sample_time_power"]
    high = progress <= high_steps
    times = np.empty_like(progress)
    hr = (1.0 - progress[high] / high_steps).clip(0.0, 1.0)
    lr = ((1.0 - progress[~high]) / low_steps).clip(0.0, 1.0)
    bnd = cfg["time_schedule_boundary"]
    times[high] = bnd + (cfg["time_max"] - bnd) * hr ** high_power
    times[~high] = cfg["time_min"] + (bnd - cfg["time_min"]) * lr ** low_power
    return np.append(times, 0.0).tolist()


def churn_plan(cfg: dict, t: float):
    """The scalar part of ``_apply_forward_pinned_churn`` (ecsi.py:670-732): None when the step does not churn, else
    (t_hat, a, b, c) with x_hat = a x_t + b x_T + c noise."""
    if not cfg["churn_end_time"] < t < cfg["time_max"]:
        return None
    span = cfg["time_max"] - cfg["churn_end_time"]
    weight = ((t - cfg["churn_end_time"]) / span) ** 2
    lo, hi = cfg["churn_factor_range"]
    chi = lo + (hi - lo) * weight
    if chi <= 0.0:
        return None
    C = Coeffs(cfg["gamma_max"])
    sigma = float(C.sigma_eff(t))
    target = (1.0 + chi) * sigma
    if target <= sigma:
        return None
    if target >= float(C.sigma_eff(cfg["time_max"])):
        t_hat = cfg["time_max"]
    else:
        low, high = t, cfg["time_max"]
        for _ in range(60):
            mid = 0.5 * (low + high)
            if float(C.sigma_eff(mid)) < target:
                low = mid
            else:
                high = mid
        t_hat = high
    if t_hat <= t:
        return None
    ratio = float(C.alpha(t_hat)) / _clip(float(C.alpha(t)))
    variance = float(C.gamma(t_hat)) ** 2 - (ratio ** 2) * float(C.gamma(t)) ** 2
    if variance <= 0.0:
        return None
    return t_hat, ratio, float(C.beta(t_hat)) - ratio * float(C.beta(t)), math.sqrt(variance)


def update_plan(cfg: dict, t: float, t_next: float):
    """``_update_step`` (ecsi.py:734-807) as a linear form: x_next = A x_t + B x0_hat + C x_T + D noise.
    SI ODE at or below sde_end_time, ECSI SDE above (the choice of ecsi.py:540-550); D = 0 means no draw."""
    C_ = Coeffs(cfg["gamma_max"])
    a_t, b_t = C_.alpha(t), C_.beta(t)
    ss = cfg["step_scale"]
    if t <= cfg["sde_end_time"]:
        a_n, b_n = C_.alpha(t_next), C_.beta(t_next)
        c_skip = b_n / b_t
        c_upd = a_n - a_t * c_skip
        # x + ss (c_skip x + c_upd x0 - x)
        return 1.0 + ss * (c_skip - 1.0), ss * c_upd, 0.0, 0.0
    g, gd = C_.gamma(t), C_.gamma_deriv(t)
    eps = cfg["eta"] * (g * gd + g ** 2 / _clip(a_t))
    k = (gd + eps / _clip(g)) / _clip(g)          # drift = -x0 + xT + k (x - a x0 - b xT)
    dt = t - t_next
    return 1.0 - ss * dt * k, -ss * dt * (-1.0 - k * a_t), -ss * dt * (1.0 - k * b_t), _sqrt(2 * eps * dt)


# ----------------------------------------------------------------------------- geometry
def quaternion_to_matrix(q: torch.Tensor) -> torch.Tensor:
    """utils/geometry/random_augment.py:317-350."""
    r, i, j, k = q.unbind(-1)
    two_s = 2.0 / (q * q).sum(-1)
    o = torch.stack((1 - two_s * (j * j + k * k), two_s * (i * j - k * r), two_s * (i * k + j * r),
                     two_s * (i * j + k * r), 1 - two_s * (i * i + k * k), two_s * (j * k - i * r),
                     two_s * (i * k - j * r), two_s * (j * k + i * r), 1 - two_s * (i * i + j * j)), -1)
    return o.reshape(q.shape[:-1] + (3, 3))


def random_rotations(shape, rng) -> torch.Tensor:
    """``random_rotations_torch`` (random_augment.py:296-314): normalised normal quaternions, real part made positive."""
    n = math.prod(shape)
    o = rng.randn((n, 4))
    s = (o * o).sum(1)
    q = o / torch.copysign(torch.sqrt(s), o[:, 0])[:, None]
    return quaternion_to_matrix(q).reshape(*shape, 3, 3)


def random_augmentation(coords: list, mask: torch.Tensor, rng, s_trans: float = 1.0) -> list:
    """``CenterRandomAugmentation._augment`` with centering=False (random_augment.py:463-513): one rotation and one
    translation per coordinate set, shared by all tensors of `coords`; padding atoms set to zero."""
    ref = coords[0]
    R = random_rotations(tuple(ref.shape[:-2]), rng)
    out = [torch.einsum("...md,...ds->...ms", x, R) for x in coords]
    trans = rng.randn(tuple(ref[..., 0:1, :].shape)) * s_trans
    out = [x + trans for x in out]
    mb = mask.bool().unsqueeze(-1)
    return [x.masked_fill(~mb, 0.0) for x in out]


def do_centering(coords: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """random_augment.py:90-130 with mask_to_zero=True."""
    mb = mask.bool().unsqueeze(-1)
    safe = coords.masked_fill(~mb, 0.0)
    total = mask.sum(-1, keepdim=True).clamp(1)
    center = safe.sum(-2, keepdim=True) / total[..., None]
    return (coords - center).masked_fill(~mb, 0.0)


def rigid_transform(coords: torch.Tensor, target: torch.Tensor, weights: torch.Tensor, eps: float = 1e-8):
    """``get_rigid_transform_torch`` (utils/geometry/rigid_align.py:685-771): weighted Kabsch, returns (R^T, t)."""
    w_sum = weights.sum(-1) + eps
    cc = (coords * weights[..., None]).sum(-2) / w_sum[..., None]
    tc = (target * weights[..., None]).sum(-2) / w_sum[..., None]
    c0, t0 = coords - cc[..., None, :], target - tc[..., None, :]
    H = torch.einsum("...ni,...nj->...ij", c0 * weights[..., None], t0)
    U, _, Vh = torch.linalg.svd(H)
    F = torch.eye(3).tile(*H.shape[:-2], 1, 1)
    F[..., -1, -1] = torch.sign(torch.linalg.det(U @ Vh))
    RT = U @ F @ Vh
    t = (tc[..., None, :] - cc[..., None, :] @ RT).squeeze(-2)
    return RT, t


def custom_rigid_align(coords, target, mask, rotation_only: bool = False):
    """ecsi.py:59-103 with output_mask = mask."""
    mb = mask.bool().unsqueeze(-1)
    coords, target = coords.float(), target.float()
    RT, T = rigid_transform(coords.masked_fill(~mb, 0.0), target.masked_fill(~mb, 0.0), mask.float().expand(coords.shape[:-1]))
    out = coords.masked_fill(~mb, 0.0) @ RT
    if not rotation_only:
        out = (out + T.unsqueeze(-2)).masked_fill(~mb, 0.0)
    return out


# ----------------------------------------------------------------------------- the loop
def sample_loop(x_apo, atom_mask, step_fn, s_inputs, num_steps: int, num_samples: int, rng, cfg: dict | None = None,
                single_conditioning=None):
    """ecsi.py:498-560 (after the time-independent precompute) with ``sample_prior`` (:562-587).

    x_apo (B, Nprior, La, 3) prior coordinates; atom_mask (B, La); ``step_fn(r_noisy (B,N,La,6), s (B,1,Lt,c_s)) ->
    r_update (B,N,La,3)`` is the score network; ``single_conditioning(s_inputs, c_noise (1,1)) -> s``.
    Returns (x_T, x_final)."""
    cfg = dict(DEFAULTS, **(cfg or {}))
    times = sampling_schedule(cfg, num_steps)
    mask = atom_mask[..., None, :]
    idx = [i % x_apo.shape[1] for i in range(num_samples)]
    (x_T,) = random_augmentation([x_apo[:, idx].float()], mask, rng)
    x_t = x_T.clone()
    for step in range(num_steps):
        x_t, x_T = random_augmentation([x_t, x_T], mask, rng)
        t, t_next = times[step], times[step + 1]
        plan = churn_plan(cfg, t)
        x_noisy = x_t
        if plan is not None:
            t, a, b, c = plan
            noise = rng.randn(tuple(x_t.shape)).masked_fill(~mask[..., None], 0.0)
            x_noisy = a * x_t + b * x_T + c * noise
        c_in, c_skip, c_out = bridge_scalings(cfg, t)
        s = single_conditioning(s_inputs, torch.tensor(c_noise(t)).view(1, 1))
        r = torch.cat([c_in * x_noisy, x_T / cfg["sigma_T"]], dim=-1)
        x0 = c_skip * x_noisy + c_out * step_fn(r, s)
        x0 = custom_rigid_align(x0, x_noisy, mask, rotation_only=True)
        x0 = do_centering(x0, mask)
        A, B, C, D = update_plan(cfg, t, t_next)
        x_t = A * x_noisy + B * x0 + C * x_T
        if D != 0.0:
            x_t = x_t + D * rng.randn(tuple(x_noisy.shape)).masked_fill(~mask[..., None], 0.0)
    return x_T, x_t


def diffusion_step_fn(q, c, p, token_index, atom_mask, pair_bias, token_mask, w: dict, atom_heads: int, atom_blocks: int,
                      token_heads: int, token_blocks: int, mode: str = "fp32"):
    """The score network as the oracle states it (pairformer_oracle.diffusion_step), closed over a complex's tensors."""
    def step(r_noisy, s):
        return O.diffusion_step(r_noisy, q, c, p, token_index, atom_mask, s, pair_bias, token_mask, w, atom_heads, atom_blocks,
                                token_heads, token_blocks, mode)
    return step
