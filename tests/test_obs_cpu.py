"""Profiler selection, tensor dumps, seeding and FLOP accounting."""
import json
import os
import types

import torch

from mindspeed_rl_b200.obs.profiler import (TensorDump, num_floating_point_operations, profiler_start, profiler_step,
                                            profiler_stop, range_timer, seed_all)


def _cfg(tmp, **kw):
    base = dict(profile=True, mstx=False, stage="all", profile_save_path=str(tmp), profile_export_type="db",
                profile_level="level0", profile_with_memory=False, profile_with_cpu=True, profile_with_module=False,
                profile_record_shapes=False, profile_step_start=1, profile_step_end=2, profile_ranks="all")
    base.update(kw)
    return types.SimpleNamespace(**base)


def test_profiler_selection_and_trace(tmp_path):
    assert profiler_start(None, "actor_update") is None
    assert profiler_start(_cfg(tmp_path, profile=False), "actor_update", 1) is None
    assert profiler_start(_cfg(tmp_path, stage="actor_generate"), "actor_update", 1) is None
    assert profiler_start(_cfg(tmp_path, profile_ranks=[3]), "actor_update", 1) is None
    assert profiler_start(_cfg(tmp_path), "actor_update", 5) is None          # outside the step window
    prof = profiler_start(_cfg(tmp_path, stage=["actor_update"]), "actor_update", 1)
    assert prof is not None
    torch.randn(64, 64) @ torch.randn(64, 64)
    profiler_step(prof)
    profiler_stop(prof)
    files = os.listdir(tmp_path / "actor_update")
    assert any(f.endswith(".json") for f in files)


def test_range_timer_is_transparent():
    @range_timer
    def f(x):
        return x + 1
    assert f(1) == 2 and f.__name__ == "f"


def test_tensor_dump(tmp_path):
    cfg = types.SimpleNamespace(msprobe=True, dump_path=str(tmp_path), key_data_dump=True, step_start=0, step_end=0)
    d = TensorDump(cfg, save_values=True)
    d.save_data("actor_update", {"logp": torch.tensor([1.0, -3.0, float("nan")]), "n": 3, "skip": object()})
    d.step()
    rec = json.load(open(tmp_path / "step0" / "rank0" / "actor_update.json"))
    assert rec["logp"]["nan"] == 1 and rec["logp"]["shape"] == [3] and rec["n"] == 3 and "skip" not in rec
    assert torch.load(tmp_path / "step0" / "rank0" / "actor_update.pt")["logp"].shape == (3,)
    d.save_data("actor_update", {"x": torch.ones(2)})                          # iteration 1 is outside the window
    d.step()
    assert not (tmp_path / "step1").exists()
    d.save_configs({"a": types.SimpleNamespace(k=1)})
    assert json.load(open(tmp_path / "configurations.json"))["a"]["k"] == 1


def test_seed_all_reproducible():
    seed_all(7)
    a = torch.rand(3)
    seed_all(7)
    assert torch.equal(a, torch.rand(3))


def test_flops_dense_matches_closed_form():
    cfg = types.SimpleNamespace(hidden_size=64, num_layers=2, num_attention_heads=4, num_query_groups=2, kv_channels=16,
                                ffn_hidden_size=128, padded_vocab_size=1000, swiglu=True, seq_length=32)
    s, h = 32, 64
    attn = 2 * h * (64 + 2 * 32) + 2 * 64 * h + 4 * s * 64
    mlp = 2 * 3 * h * 128
    want = 3.0 * 5 * s * (2 * (attn + mlp) + 2 * h * 1000)
    assert num_floating_point_operations(cfg, 5) == want
    moe = types.SimpleNamespace(**vars(cfg), num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=32,
                                n_shared_experts=1, first_k_dense_replace=1)
    assert num_floating_point_operations(moe, 5) != want


def test_stage_boundary_raises_when_a_kernel_wait_gave_up():
    """A worker stage ends with a look at the device status words: a code left by a bounded wait
    turns into an exception at the stage boundary (injected here by writing the word on the host)."""
    import pytest
    import torch

    from mindspeed_rl_b200.ops import gemm
    from mindspeed_rl_b200.workers.base_worker import check_device_status, profiled_stage

    class W:
        @profiled_stage("actor_update")
        def update(self):
            return 7

    dev = torch.device("cpu")
    word = gemm._status_word(dev)
    try:
        assert W().update() == 7
        word.fill_(3)
        with pytest.raises(gemm.KernelTimeout, match="actor_update"):
            W().update()
        assert int(word.item()) == 0                      # the word is re-armed for the next stage
        check_device_status("again")
    finally:
        gemm._status.pop(dev, None)
