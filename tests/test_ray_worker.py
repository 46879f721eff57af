"""RayWorker against an in-process stand-in for the `ray` API (the package itself is optional)."""

import types

import pytest
import torch

from telefuser_b200.core.base_stage import BaseStage
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.worker import ray_worker


class _Ref:
    def __init__(self, fn):
        self.fn, self.done, self.value = fn, False, None


class _Method:
    def __init__(self, bound):
        self.bound = bound

    def remote(self, *a, **k):
        return _Ref(lambda: self.bound(*a, **k))


class _Actor:
    def __init__(self, obj):
        self._obj = obj

    def __getattr__(self, name):
        return _Method(getattr(self._obj, name))


def _fake_ray(log):
    mod = types.SimpleNamespace()
    mod.init = lambda **kw: log.append(("init", kw))

    def remote(cls):
        def options(**res):
            log.append(("options", res))
            return types.SimpleNamespace(remote=lambda *a, **k: _Actor(cls(*a, **k)))

        return types.SimpleNamespace(options=options)

    def get(ref):
        if not ref.done:
            ref.value, ref.done = ref.fn(), True
        return ref.value

    mod.remote, mod.get, mod.kill = remote, get, lambda actor: log.append(("kill", actor))
    return mod


class _Stage(BaseStage):
    def __init__(self):
        super().__init__("double", ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32))
        self.model_names = []

    def process(self, x, scale=2):
        if scale < 0:
            raise ValueError("negative scale")
        return x * scale


def test_ray_worker_with_stub(monkeypatch):
    monkeypatch.setattr(ray_worker, "ray", None)
    with pytest.raises(ImportError):
        ray_worker.create_ray_worker(_Stage())
    log = []
    monkeypatch.setattr(ray_worker, "ray", _fake_ray(log))
    stage = _Stage()
    stage.model_runtime_config.ray_config.num_cpus = 2
    handle = ray_worker.create_ray_worker(stage)
    assert log[0][0] == "init" and log[1] == ("options", {"num_cpus": 2, "memory": 32 * 1024**3, "num_gpus": 0})
    assert torch.equal(handle.process(torch.ones(2)), torch.full((2,), 2.0))
    waiter = handle.process_async(torch.ones(2), scale=3)
    assert torch.equal(waiter(), torch.full((2,), 3.0))
    with pytest.raises(ValueError):
        handle.process(torch.ones(1), scale=-1)
    status = handle.get_status()
    assert status["worker_id"] == "double" and status["worker_type"] == "_Stage"
    handle.close()
    assert log[-1][0] == "kill"
