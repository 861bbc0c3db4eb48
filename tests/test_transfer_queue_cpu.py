"""TransferQueue: codec, shards over ZeroMQ, TD-equivalent adapter, GRPO end-to-end on it."""
import torch

from mindspeed_rl_b200.data.transfer_dock import GRPOTransferDock
from mindspeed_rl_b200.data.transfer_queue import (DataStrategy, SyncTransferQueueAdapter, TransferQueueClient,
                                                   TransferQueueShard, decode_tensor_list, encode_tensor_list)


def test_codec_round_trip():
    ts = [torch.arange(7, dtype=torch.int32), torch.randn(3, 5), torch.randn(4).bfloat16(), None,
          torch.tensor([True, False, True]), torch.zeros(0, dtype=torch.int64), torch.tensor(3.5)]
    back = decode_tensor_list(encode_tensor_list(ts))
    assert len(back) == len(ts)
    for a, b in zip(ts, back):
        if a is None:
            assert b is None
        else:
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)


def test_shards_and_client_blocking_get():
    import threading
    import time

    shards = [TransferQueueShard(i, 3, timeout_s=10) for i in range(3)]
    client = TransferQueueClient([s.address for s in shards])
    idx = [0, 1, 2, 3, 4, 7]
    data = {"a": [torch.full((i + 1,), i, dtype=torch.int32) for i in idx], "b": [torch.randn(2, 2) for _ in idx]}
    got = {}

    def reader():                                      # asks before the rows exist
        got.update(TransferQueueClient([s.address for s in shards]).get(["a", "b"], [7, 0, 3]))

    t = threading.Thread(target=reader)
    t.start()
    time.sleep(0.1)
    client.put(data, idx)
    t.join(10)
    assert not t.is_alive()
    assert [int(x[0]) for x in got["a"]] == [7, 0, 3] and torch.equal(got["b"][1], data["b"][0])
    assert sorted(shards[1].rows["a"]) == [1, 4, 7]
    client.clear([1, 4])
    assert sorted(shards[1].rows["a"]) == [7]
    client.clear(None)
    assert all(not s.rows for s in shards)
    for s in shards:
        s.shutdown()


def _fill(store, n_prompts=4, n=2):
    from mindspeed_rl_b200.data.transfer_dock import put_prompts_experience
    batch = {"prompts": [torch.arange(3 + i) for i in range(n_prompts)]}
    data, idx = put_prompts_experience(batch, n)
    store.put_experience(data, idx, is_prompt=True)
    return idx


def test_adapter_matches_transfer_dock():
    td = GRPOTransferDock(4, 2)
    strategy = DataStrategy("transfer_queue", num_shards=2)
    manager, desc = strategy.create(4, 2)
    tq = DataStrategy.attach(manager, desc)
    assert isinstance(tq, SyncTransferQueueAdapter) and DataStrategy("td").create(4, 2)[1] is None
    for store in (td, tq):
        _fill(store)
    b1, i1 = td.get_experience("actor_rollout", ["prompts", "prompt_length"], 4)
    b2, i2 = tq.get_experience("actor_rollout", ["prompts", "prompt_length"], indexes=i1)   # same rows (sampling is random)
    assert i1 == i2 and all(torch.equal(b1[k], b2[k]) for k in b1)
    resp = {"responses": [torch.arange(5 + j, dtype=torch.int64) for j in range(4)],
            "response_length": [torch.tensor([5 + j]) for j in range(4)]}
    for store in (td, tq):
        store.put_experience(resp, i1)
    for store in (td, tq):
        assert not store.all_consumed("actor_rollout")
    b1, j1 = td.get_experience("actor_train", ["responses", "response_length"], 2, get_n_samples=True)
    b2, j2 = tq.get_experience("actor_train", ["responses", "response_length"], indexes=j1)
    assert j1 == j2 and all(torch.equal(b1[k], b2[k]) for k in b1)
    assert tq.get_experience("actor_train", ["rm_scores"], 2) == (None, None)      # nothing ready
    tq.update_metrics("x", value=[1.0], cumulate=True)
    tq.clear()
    assert tq.get_experience("actor_rollout", ["prompts"], 4) == (None, None)
    for s in strategy.shards:
        s.shutdown()


def test_grpo_end_to_end_on_transfer_queue():
    from test_e2e_grpo_cpu import build
    from mindspeed_rl_b200.datasets.synthetic import SyntheticPromptLoader
    from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer
    from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
    from mindspeed_rl_b200.workers.rule_reward import RuleReward

    torch.manual_seed(0)
    actor, rl, gen = build(n_prompts=4, n_samples=2, max_tokens=16, iters=1)
    rl.data_strategy, rl.transfer_queue_data_shard_num = "tq", 2
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=1, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=4, n_samples_per_prompt=2, pad_token_id=0)
    assert isinstance(trainer.transfer_dock, SyncTransferQueueAdapter)
    hist = trainer.fit(iter(SyntheticPromptLoader(4, 32, 1024, seed=0)))
    assert len(hist) == 1 and hist[0]["timing/update"] > 0 and "actor/pg_loss" in hist[0]
