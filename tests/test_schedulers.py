"""Schedulers: flow-match sigma schedules / Euler step, UniPC exactness and convergence order."""
import torch

from telefuser_b200.schedulers.flow_match import FlowMatchScheduler, schedule_wan, schedule_wan_mix
from telefuser_b200.schedulers.unipc import FlowUniPCMultistepScheduler


def test_wan_schedule_values_and_step():
    s, t = schedule_wan(4, shift=5.0)
    raw = torch.linspace(1, 0, 5)[:-1]
    assert torch.allclose(s, 5 * raw / (1 + 4 * raw)) and torch.allclose(t, s * 1000)
    sch = FlowMatchScheduler("Wan")
    sch.set_timesteps(4, shift=5.0)
    x, v = torch.ones(2, 3), torch.full((2, 3), 2.0)
    out = sch.step(v, sch.timesteps[1], x)
    assert torch.allclose(out, x + v * (sch.sigmas[2] - sch.sigmas[1]))
    last = sch.step(v, sch.timesteps[3], x)
    assert torch.allclose(last, x + v * (0 - sch.sigmas[3]))
    assert torch.allclose(sch.step_with_guidance(v, v * 0, 1.0, sch.timesteps[1], x), out)
    noisy = sch.add_noise(x, v, sch.timesteps[2])
    assert torch.allclose(noisy, (1 - sch.sigmas[2]) * x + sch.sigmas[2] * v)


def test_other_templates_are_monotone_and_mix_joins_at_boundary():
    for name, kw in (("FLUX.1", {}), ("Qwen-Image", {"dynamic_shift_len": 4096}), ("FLUX.2", {}), ("Z-Image", {}),
                     ("LTX.2", {})):
        sch = FlowMatchScheduler(name)
        sch.set_timesteps(8, **kw)
        assert (sch.sigmas[:-1] >= sch.sigmas[1:]).all(), name
    s, t = schedule_wan_mix((6, 6), shift=(3.0, 8.0), boundary=0.875)
    assert (s[:-1] >= s[1:]).all() and (t[s >= 0.875] >= 875).all()


def _integrate(sched, steps, x1, x0_fn, stop_fraction=1.0):
    sched.set_timesteps(steps, shift=3.0)
    x = x1.clone()
    for i, t in enumerate(sched.timesteps[: int(steps * stop_fraction)]):
        sigma = sched.sigmas[i]
        x0 = x0_fn(x, sigma)
        v = (x - x0) / sigma
        x = sched.step(v, t, x)[0]
    return x


def test_unipc_is_exact_for_constant_data_prediction():
    target = torch.tensor([[0.3, -1.2, 2.0]])
    out = _integrate(FlowUniPCMultistepScheduler(), 6, torch.randn(1, 3), lambda x, s: target)
    assert torch.allclose(out, target, atol=1e-5)


def test_unipc_second_order_beats_first_order_at_a_fixed_noise_level():
    # Stop half-way (same sigma for every even step count) so the final jump to sigma = 0, which is
    # first order by construction, does not mask the multistep order.
    c = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    x1 = torch.tensor([[0.5, 0.5]], dtype=torch.float64)
    fn = lambda x, s: 0.6 * torch.tanh(x) + c * (1 - 0.5 * s)  # noqa: E731
    ref = _integrate(FlowUniPCMultistepScheduler(solver_order=2), 400, x1, fn, 0.5)
    err = {o: [(_integrate(FlowUniPCMultistepScheduler(solver_order=o), n, x1, fn, 0.5) - ref).abs().max().item()
               for n in (8, 16, 32)] for o in (1, 2)}
    assert err[2][2] < err[1][2] * 0.2
    assert err[2][2] < err[2][1] * 0.4  # better than halving per doubling of steps


def test_unipc_add_noise_and_timesteps():
    s = FlowUniPCMultistepScheduler()
    s.set_timesteps(1000, shift=10.0)
    assert len(s.timesteps) == 1000 and len(s.sigmas) == 1001 and float(s.sigmas[-1]) == 0.0
    x, n = torch.ones(1, 2, 2), torch.zeros(1, 2, 2)
    t = s.timesteps[358].view(1)
    sig = s.sigmas[s.index_for_timestep(t[0])]
    assert abs(float(sig) - float(s.sigmas[358])) < 2e-3
    assert torch.allclose(s.add_noise(x, n, t), (1 - sig) * x)


def _reference_flow_match():
    """The reference's scheduler file, loaded by path (its package `__init__` needs packages that are not installed)."""
    import importlib.util
    from pathlib import Path

    import pytest

    path = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "telefuser" / "schedulers" / "flow_match.py"
    if not path.is_file():
        pytest.skip("the reference tree is not installed")
    spec = importlib.util.spec_from_file_location("telefuser_ref_flow_match_for_tests", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.FlowMatchScheduler


def test_every_template_equals_the_reference_schedule():
    Ref = _reference_flow_match()
    cases = [("Wan", {"shift": 5.0}), ("Wan", {"shift": 3.0, "denoising_strength": 0.6}), ("FLUX.1", {}),
             ("FLUX.1", {"shift": 2.0}), ("Qwen-Image", {"dynamic_shift_len": 4096}),
             ("Qwen-Image", {"dynamic_shift_len": 1024, "denoising_strength": 0.8}), ("FLUX.2", {"dynamic_shift_len": 4096}),
             ("Z-Image", {}), ("Z-Image", {"shift": 6.0}), ("LTX.2", {})]  # fmt: skip
    torch.manual_seed(0)
    for name, kw in cases:
        for steps in (4, 20):
            try:
                want = Ref(name)
                want.set_timesteps(steps, **kw)
            except TypeError:
                continue  # the reference's template does not take this keyword
            got = FlowMatchScheduler(name)
            got.set_timesteps(steps, **kw)
            assert torch.equal(got.sigmas.float(), want.sigmas.float()), (name, kw, steps)
            assert torch.equal(got.timesteps.float(), want.timesteps.float()), (name, kw, steps)
            x, v = torch.randn(2, 5), torch.randn(2, 5)
            for i in (0, steps // 2, steps - 1):
                a, b = got.step(v, got.timesteps[i], x), want.step(v, want.timesteps[i], x)
                assert torch.allclose(a, b, atol=1e-6, rtol=0), (name, kw, steps, i)
