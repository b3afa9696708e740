"""K-Fold's sampler loop on the B200 kernels: ``KFoldECSI.sample_structure`` (model/modules/ecsi.py:182-808, inference part).

Same class name, configuration fields, method names and arguments as the reference's ECSI bridge sampler.  The host keeps
what the reference keeps on the host -- the time schedule, the bridge, churn and update coefficients (plain floats) -- and
draws the normals in the reference's order (rotation quaternions, translation, churn noise, update noise), so that a run
started from the same generator state on the same device consumes the same numbers as the reference's torch backend.
Everything that touches coordinates runs in three small kernels per step (``kfb_coords_augment``, ``kfb_sampler_prepare``,
``kfb_sampler_update``) around the score network (``modules.DiffusionStack.step``), which can be replayed as a CUDA graph.

The time-independent precompute of the reference (pair conditioning, atom embedder: model/modules/ecsi.py:503-505) is
outside the accelerated path: pass its results as ``precomputed=dict(q=..., c=..., p=..., pair_bias=...)`` or give a
``score_model`` that implements ``get_pair_conditioning`` / ``get_atom_embeddings``.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

from . import functional as F
from .graphs import GraphedCall

__all__ = ["KFoldECSI", "SICoeffs", "custom_rigid_align", "do_centering", "CenterRandomAugmentation"]


def _clip(t: float, eps: float = 1e-10) -> float:
    return max(t, eps)


def _sqrt(t: float) -> float:
    return max(t, 0.0) ** 0.5


@dataclasses.dataclass
class SICoeffs:
    """Stochastic-interpolant coefficients (model/modules/ecsi.py:106-131): linear route, gamma^2 = 4 gamma_max^2 t (1 - t)."""

    gamma_max: float

    def alpha(self, t: float) -> float:
        return 1.0 - t

    def beta(self, t: float) -> float:
        return t

    def gamma(self, t: float) -> float:
        return 2 * self.gamma_max * _sqrt(t * (1 - t))

    def gamma_deriv(self, t: float) -> float:
        return self.gamma_max * (1 - 2 * t) / _clip(_sqrt(t * (1 - t)))

    def sigma_eff(self, t: float) -> float:
        return self.gamma(t) / _clip(self.alpha(t))


# ----------------------------------------------------------------------------- geometry helpers with the reference's names
def custom_rigid_align(coords: torch.Tensor, target: torch.Tensor, mask: torch.Tensor | None, rotation_only: bool = False,
                       output_mask: torch.Tensor | None = None) -> torch.Tensor:
    """Weighted rigid alignment (model/modules/ecsi.py:59-103).  ``output_mask`` other than ``mask`` is not available."""
    if output_mask is not None and output_mask is not mask:
        raise NotImplementedError("custom_rigid_align: a separate output_mask is not available")
    if mask is None:
        mask = torch.ones(coords.shape[:-1], dtype=torch.bool, device=coords.device)
    return F.rigid_align(coords, target, mask, rotation_only=rotation_only)


def do_centering(coords: torch.Tensor, mask: torch.Tensor, mask_to_zero: bool = True) -> torch.Tensor:
    """utils/geometry/random_augment.py:90-130 (the mask_to_zero form the sampler uses)."""
    if not mask_to_zero:
        raise NotImplementedError("do_centering: only the mask_to_zero form is available")
    return F.center_coords(coords, mask)


class _TorchNormals:
    """Standard normals from the device's default generator, drawn with the calls the reference makes."""

    def __init__(self, device):
        self.device = device

    def randn(self, shape) -> torch.Tensor:
        return torch.randn(tuple(shape), dtype=torch.float32, device=self.device)


class CenterRandomAugmentation:
    """Random rotation and translation of coordinate sets (utils/geometry/random_augment.py:353-513), centering off (the
    form the sampler uses), padding atoms set to zero.  ``rng.randn(shape)`` supplies the normals: first (n, 4) for the
    quaternions, then (*, 1, 3) for the translation."""

    def __init__(self, s_trans: float = 1.0):
        self.s_trans = s_trans

    def __call__(self, *coords: torch.Tensor, mask: torch.Tensor, rng=None, centering: bool = False):
        if centering:
            raise NotImplementedError("CenterRandomAugmentation: the sampler calls it with centering=False; that form is built")
        ref = coords[0]
        rng = rng or _TorchNormals(ref.device)
        n = math.prod(ref.shape[:-2])
        normals = rng.randn((n, 4)).to(ref.device)
        trans = None
        if self.s_trans > 0.0:
            trans = rng.randn(tuple(ref[..., 0:1, :].shape)).to(ref.device) * self.s_trans
        out = F.coords_augment([x.float() for x in coords], normals, trans, mask)
        return out[0] if len(out) == 1 else tuple(out)


class KFoldECSI:
    """Endpoint-conditioned stochastic-interpolant sampler (model/modules/ecsi.py:182-808), inference part."""

    @dataclasses.dataclass(kw_only=True)
    class Config:
        """The inference fields of the reference's ``KFoldECSI.Config`` (ecsi.py:205-300), same names and defaults."""

        sigma_0: float = 16.0
        sigma_T: float = 27.0
        cov_0T: float = 175.0
        time_min: float = 1e-8
        time_max: float = 0.9999
        gamma_max: float = 6.0
        time_schedule_boundary: float = 0.5
        sample_step_fraction: tuple = (0.4, 0.6)
        sample_time_power: tuple = (0.5, 2.0)
        sde_end_time: float = 0.1
        eta: float = 1.0
        step_scale: float = 1.0
        churn_end_time: float = 0.5
        churn_factor_range: tuple = (0.1, 0.4)

        def __post_init__(self) -> None:
            schedules = (self.sample_step_fraction, self.sample_time_power)
            if any(len(v) != 2 for v in schedules):
                raise ValueError("Sampling schedule tuples must each contain exactly two values.")
            if any(not math.isfinite(x) or x <= 0 for v in schedules for x in v):
                raise ValueError("Sampling schedule values must be finite and positive.")
            if not math.isclose(sum(self.sample_step_fraction), 1.0, rel_tol=0.0, abs_tol=1e-8):
                raise ValueError("Sampling step fractions must sum to one.")
            if not self.time_min < self.time_schedule_boundary < self.time_max:
                raise ValueError("time_schedule_boundary must lie between time_min and time_max.")
            if len(self.churn_factor_range) != 2 or any(not math.isfinite(x) or x < 0 for x in self.churn_factor_range):
                raise ValueError("churn_factor_range must contain two finite non-negative values.")

    def __init__(self, cfg: "KFoldECSI.Config", score_model):
        """``score_model``: an object with ``get_single_conditioning``, ``get_pair_bias`` and ``step`` -- a
        ``kfold_b200.modules.DiffusionStack`` or anything with the reference's ``DiffusionModule`` interface."""
        self.cfg = cfg
        self.score_model = score_model
        self.random_augmentation = CenterRandomAugmentation()
        self.coeff = SICoeffs(cfg.gamma_max)
        for k, v in dataclasses.asdict(cfg).items():
            setattr(self, k, v)

    # ------------------------------------------------------------------ scalar schedule (host floats, as in the reference)
    def _get_bridge_scalings(self, t: float):
        """ecsi.py:373-417."""
        C = self.coeff
        a, b, g = C.alpha(t), C.beta(t), C.gamma(t)
        s0, sT, cov = self.sigma_0, self.sigma_T, self.cov_0T
        c_in = 1 / _clip(_sqrt((a * s0) ** 2 + (b * sT) ** 2 + 2 * a * b * cov + g ** 2))
        c_skip = (a * s0 ** 2 + b * cov) * (c_in ** 2)
        c_out = _sqrt((b * s0 * sT) ** 2 - (b * cov) ** 2 + g ** 2 * s0 ** 2) * c_in
        return c_in, c_skip, c_out

    def c_noise(self, t: float) -> float:
        return 0.25 * math.log(_clip(t, 1e-10))

    def get_sampling_schedule(self, num_steps: int) -> list:
        """ecsi.py:438-466: strictly decreasing times ending at zero, length num_steps + 1."""
        if num_steps < 1:
            raise ValueError("num_steps must be positive.")
        progress = np.linspace(0.0, 1.0, num_steps)
        high_steps, low_steps = self.sample_step_fraction
        high_power, low_power = self.sample_time_power
        high = progress <= high_steps
        times = np.empty_like(progress)
        hr = (1.0 - progress[high] / high_steps).clip(0.0, 1.0)
        lr = ((1.0 - progress[~high]) / low_steps).clip(0.0, 1.0)
        bnd = self.time_schedule_boundary
        times[high] = bnd + (self.time_max - bnd) * hr ** high_power
        times[~high] = self.time_min + (bnd - self.time_min) * lr ** low_power
        times = np.append(times, 0.0)
        if np.any(times[:-1] <= times[1:]):
            raise RuntimeError("ECSI sampling schedule must decrease.")
        return times.tolist()

    def _churn_plan(self, t: float):
        """The host part of ``_apply_forward_pinned_churn`` (ecsi.py:670-732): None when the step does not churn, else
        (t_hat, a, b, c) with x_hat = a x_t + b x_T + c noise."""
        if not self.churn_end_time < t < self.time_max:
            return None
        span = self.time_max - self.churn_end_time
        weight = ((t - self.churn_end_time) / span) ** 2
        lo, hi = self.churn_factor_range
        chi = lo + (hi - lo) * weight
        if chi <= 0.0:
            return None
        C = self.coeff
        sigma = float(C.sigma_eff(t))
        target = (1.0 + chi) * sigma
        if target <= sigma:
            return None
        if target >= float(C.sigma_eff(self.time_max)):
            t_hat = self.time_max
        else:
            low, high = t, self.time_max
            for _ in range(60):      # invert the monotonic effective-noise schedule inside the churn band
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

    def _update_plan(self, t: float, t_next: float, mode: str, equation: str):
        """``_update_step`` (ecsi.py:734-807) as x_next = A x_t + B x0_hat + C x_T + D noise."""
        if mode not in {"ode", "sde"}:
            raise ValueError(f"Unknown sampler mode: {mode!r}.")
        if equation not in {"si", "ecsi"}:
            raise ValueError(f"Unknown sampler equation: {equation!r}.")
        C = self.coeff
        a_t, b_t, ss = C.alpha(t), C.beta(t), self.step_scale
        if mode == "ode":
            a_n, b_n = C.alpha(t_next), C.beta(t_next)
            if equation == "si":
                c_skip = b_n / b_t
                return 1.0 + ss * (c_skip - 1.0), ss * (a_n - a_t * c_skip), 0.0, 0.0
            g, g_n = C.gamma(t), C.gamma(t_next)
            r = g_n / _clip(g)          # x_target = a_n x0 + b_n xT + r (x - a x0 - b xT)
            return 1.0 + ss * (r - 1.0), ss * (a_n - r * a_t), ss * (b_n - r * b_t), 0.0
        g, gd = C.gamma(t), C.gamma_deriv(t)
        eps = self.eta * (g * gd + g ** 2 / _clip(a_t))
        dt = t - t_next
        D = _sqrt(2 * eps * dt)
        if equation == "si":
            f_t, s_t = 1 / _clip(b_t), -1 - a_t / _clip(b_t)
            return 1.0 - ss * dt * f_t, -ss * dt * s_t, 0.0, D
        k = (gd + eps / _clip(g)) / _clip(g)        # drift = -x0 + xT + k (x - a x0 - b xT)
        return 1.0 - ss * dt * k, -ss * dt * (-1.0 - k * a_t), -ss * dt * (1.0 - k * b_t), D

    # ------------------------------------------------------------------ steps on coordinates
    def _apply_forward_pinned_churn(self, x_t, x_T, mask, t: float, noise: torch.Tensor | None = None, rng=None):
        """ecsi.py:670-732; returns (x_hat, t_hat).  ``noise`` may be injected, as in the reference."""
        plan = self._churn_plan(t)
        if plan is None:
            return x_t, t
        t_hat, a, b, c = plan
        if noise is None:
            noise = (rng or _TorchNormals(x_t.device)).randn(tuple(x_t.shape)).to(x_t.device)
        x_hat, _ = F.sampler_prepare(x_t, x_T, mask, 1.0, self.sigma_T, churn=(a, b, c), noise=noise)
        return x_hat, t_hat

    def _update_step(self, x_t, x_0_hat, x_T, mask, t: float, t_next: float, mode: str = "ode", equation: str = "si",
                     noise: torch.Tensor | None = None, rng=None):
        """ecsi.py:734-807 on an already aligned and centred x_0_hat (the fused form lives in ``_fused_update``)."""
        A, B, C, D = self._update_plan(t, t_next, mode, equation)
        out = A * x_t + B * x_0_hat + C * x_T
        if D != 0.0:
            if noise is None:
                noise = (rng or _TorchNormals(x_t.device)).randn(tuple(x_t.shape)).to(x_t.device)
            out = out + D * noise.masked_fill(~mask[..., None], 0.0)
        return out

    def sample_prior(self, f_input, num_samples: int, rng=None) -> torch.Tensor:
        """ecsi.py:562-587: the prior (apo) coordinates cycled over the samples, randomly rotated and translated."""
        x_apo = f_input.atom.prior_coords.permute(0, 2, 1, 3)
        num_prior = x_apo.shape[-3]
        idx = [i % num_prior for i in range(num_samples)]
        x_T = x_apo[:, idx, :, :].float().contiguous()
        return self.random_augmentation(x_T, mask=f_input.atom.pad_mask.unsqueeze(-2), rng=rng)

    # ------------------------------------------------------------------ the loop
    @torch.no_grad()
    def sample_structure(self, f_input, s_inputs: torch.Tensor, z: torch.Tensor | None, num_steps: int = 100, num_samples: int = 1,
                         chunk_size: int | None = None, return_traj: bool = False, *, precomputed: dict | None = None,
                         rng=None, cuda_graph: bool = False) -> dict:
        """ecsi.py:468-560.  ``f_input``: anything with ``.atom.pad_mask / .token_index / .prior_coords`` and
        ``.token.pad_mask``.  ``precomputed``: q (B, La, c_atom), c, p (B, W, 32, 128, c_pair) and pair_bias
        (B, Nblock, H, Lt, Lt) of the time-independent precompute; without it the score model must provide
        ``get_pair_conditioning`` / ``get_atom_embeddings``.  ``rng``: source of the standard normals (``randn(shape)``),
        default the device's generator.  ``cuda_graph``: capture the score network once and replay it every step.
        ``chunk_size`` is accepted for signature compatibility; all samples go through the network together."""
        model = self.score_model
        dev = s_inputs.device
        rng = rng or _TorchNormals(dev)
        times = self.get_sampling_schedule(num_steps)
        x_T = self.sample_prior(f_input, num_samples, rng)
        x_t = x_T.clone()
        atom_mask, token_mask, token_index = f_input.atom.pad_mask, f_input.token.pad_mask, f_input.atom.token_index
        mask = atom_mask[..., None, :]
        if precomputed is not None:
            q, c, p, pair_bias = (precomputed[k] for k in ("q", "c", "p", "pair_bias"))
        else:
            zc = model.get_pair_conditioning(f_input, z)
            q, c, p = model.get_atom_embeddings(f_input, zc)
            pair_bias = model.get_pair_bias(zc)

        def network(r6: torch.Tensor, c_noise: torch.Tensor) -> torch.Tensor:
            s = model.get_single_conditioning(s_inputs, c_noise)
            return model.step(r6, q, c, p, token_index, atom_mask, s, pair_bias, token_mask)

        autocast_state = (torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda"))
        graphed = None
        traj = [x_t.cpu()] if return_traj else []
        for step in range(num_steps):
            x_t, x_T = self.random_augmentation(x_t, x_T, mask=mask, rng=rng)
            t, t_next = times[step], times[step + 1]
            plan = self._churn_plan(t)
            noise = None
            if plan is not None:
                t = plan[0]
                noise = rng.randn(tuple(x_t.shape)).to(dev)
            c_in, c_skip, c_out = self._get_bridge_scalings(t)
            x_noisy, r6 = F.sampler_prepare(x_t, x_T, mask, c_in, self.sigma_T, churn=None if plan is None else plan[1:], noise=noise)
            cn = torch.full((1, 1), self.c_noise(t), dtype=torch.float32, device=dev)
            if cuda_graph:
                if graphed is None:
                    def net(r6_, cn_):
                        with torch.autocast("cuda", enabled=autocast_state[0], dtype=autocast_state[1]):
                            return network(r6_, cn_)
                    graphed = GraphedCall(net, r6, cn)
                r_update = graphed(r6, cn)
            else:
                r_update = network(r6, cn)
            use_ode = t <= self.sde_end_time
            coef = self._update_plan(t, t_next, "ode" if use_ode else "sde", "si" if use_ode else "ecsi")
            noise = rng.randn(tuple(x_t.shape)).to(dev) if coef[3] != 0.0 else None
            x_t = F.sampler_update(x_noisy, r_update, x_T, mask, c_skip, c_out, coef, noise=noise)
            if return_traj:
                traj.append(x_t.cpu())
        out = {"init_coordinates": x_T, "coordinates": x_t}
        if return_traj:
            out["traj"] = torch.stack(traj, dim=-3)
        return out
