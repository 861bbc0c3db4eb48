"""Vision-language path on CPU: image processing, the dataset's prompt expansion and three-axis positions,
the vision-encoder worker, and a whole GRPO iteration in which rollout, reference and update read the
image embeddings the vision stage wrote."""
import numpy as np
import torch

from mindspeed_rl_b200.config import GenerateConfig, MegatronConfig, RLConfig
from mindspeed_rl_b200.config.loader import load_model_catalogue
from mindspeed_rl_b200.datasets.image_processor import ImageProcessor
from mindspeed_rl_b200.datasets.mm_utils import extend_positions, mrope_table
from mindspeed_rl_b200.datasets.multimodal_dataset import MultiModalDataset, MultiModalPromptLoader
from mindspeed_rl_b200.models.vit import VisionConfig, VisionTower

IMG, VS, VE = 1000, 1001, 1002


class _CharTokenizer:
    def tokenize(self, text):
        return [10 + (ord(c) % 200) for c in text]


def _rows(n, seed=0):
    rng = np.random.default_rng(seed)
    return [dict(prompt=f"look <image> and count {i}", images=[(rng.random((40 + 8 * (i % 3), 60, 3)) * 255).astype(np.uint8)],
                 answer=str(i)) for i in range(n)]


def _dataset(n=8):
    return MultiModalDataset(_rows(n), _CharTokenizer(), ImageProcessor(min_pixels=28 * 28, max_pixels=84 * 84),
                             image_token_id=IMG, vision_start_token_id=VS, vision_end_token_id=VE, max_prompt_length=96)


def test_dataset_expands_image_markers_and_builds_three_axis_positions():
    ds = _dataset(3)
    row = ds[0]
    ids = row["input_ids"].tolist()
    grid = row["image_grid_thw"][0].tolist()
    n_tok = grid[1] * grid[2] // 4
    assert ids.count(IMG) == n_tok and ids[ids.index(IMG) - 1] == VS and ids[ids.index(IMG) + n_tok] == VE
    assert row["pixel_values"].shape == (grid[1] * grid[2], 3 * 2 * 14 * 14)
    pos = row["position_ids"]                                   # [S, 3]
    s0 = ids.index(IMG)
    assert torch.equal(pos[:s0, 0], pos[:s0, 1]) and torch.equal(pos[:s0, 0], torch.arange(s0))
    block = pos[s0:s0 + n_tok]
    assert block[:, 0].unique().numel() == 1                    # one temporal index for a still image
    assert block[:, 1].max() - block[:, 1].min() == grid[1] // 2 - 1 and block[:, 2].max() - block[:, 2].min() == grid[2] // 2 - 1
    after = pos[s0 + n_tok]
    assert after[0] == after[1] == after[2] == block.max() + 1  # text continues after the largest position used
    ext = extend_positions(pos, 3)
    assert ext.shape[0] == pos.shape[0] + 3 and torch.equal(ext[-1], torch.full((3,), int(pos.max()) + 3))


def test_mrope_table_matches_per_axis_lookup():
    base = torch.randn(50, 16)
    pos = torch.tensor([[3, 3, 3], [4, 7, 9]])
    tab = mrope_table(pos, base, sections=(2, 3, 3))
    assert torch.equal(tab[0], base[3])                        # equal axes: the ordinary one-axis row
    assert torch.equal(tab[1, :2], base[4, :2]) and torch.equal(tab[1, 2:5], base[7, 2:5]) and torch.equal(tab[1, 5:8], base[9, 5:8])
    assert torch.equal(tab[1, 8:10], base[4, 8:10]) and torch.equal(tab[1, 13:16], base[9, 13:16])


def test_vision_tower_attends_within_an_image_only():
    cfg = VisionConfig(hidden_size=32, depth=2, num_heads=2, intermediate_size=48, out_hidden_size=24)
    tower = VisionTower(cfg, "cpu")
    p = ImageProcessor(min_pixels=28 * 28, max_pixels=56 * 56)
    a, b = _rows(2, seed=1)[0]["images"][0], _rows(2, seed=2)[1]["images"][0]
    both = p([a, b])
    alone = p([a])
    out_both = tower(both["pixel_values"], both["image_grid_thw"])
    out_alone = tower(alone["pixel_values"], alone["image_grid_thw"])
    assert out_both.shape[1] == 24 and out_both.shape[0] == sum(p.tokens_for(g) for g in both["image_grid_thw"].tolist())
    assert torch.allclose(out_both[:out_alone.shape[0]], out_alone, atol=1e-5)


def test_grpo_iteration_with_images():
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer
    from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
    from mindspeed_rl_b200.workers.rule_reward import RuleReward
    from mindspeed_rl_b200.workers.vit_worker import VitWorker

    set_parallel_state(None)
    initialize_model_parallel(1, 1, 1)
    gbs, n = 4, 2
    cat = load_model_catalogue(["tiny_qwen2"])
    actor = MegatronConfig(dict(model="tiny_qwen2", global_batch_size=gbs, micro_batch_size=2, seq_length=128, lr=1e-5,
                                lr_decay_style="constant", clip_grad=1.0, stage="ray_grpo", train_iters=2, seed=3,
                                image_token_id=IMG, vision_start_token_id=VS, vision_end_token_id=VE,
                                reset_attention_mask=True), cat)
    rl = RLConfig(dict(n_samples_per_prompt=n, mini_batch_size=gbs, clip_ratio=0.2, init_kl_coef=0.001,
                       adv_estimator="group_norm", verifier_function=["contains_token_7"], verifier_weight=[1.0],
                       actor_resource={"num_gpus": 1}, is_multimodal=True, reuse_image_embeds=True))
    gen = GenerateConfig(dict(infer_tensor_parallel_size=1, max_num_seqs=16, max_model_len=128, max_num_batched_tokens=64,
                              kv_block_size=8, enable_prefix_caching=False,
                              sampling_config=dict(max_tokens=16, temperature=1.0, top_k=-1, top_p=1.0, seed=0)))
    from mindspeed_rl_b200.config import validate_rl_args
    validate_rl_args(actor, actor, actor, rl, gen)
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker).initialize()
    vit = VitWorker(None, rl, llm_hidden_size=256, device="cpu",
                    vision_config=VisionConfig(hidden_size=32, depth=1, num_heads=2, intermediate_size=48, out_hidden_size=256))
    vit_group = SPMDWorkerGroup(vit).initialize()
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], vit_worker=vit_group, train_iters=2,
                             save_interval=0, global_batch_size=gbs, n_samples_per_prompt=n, init_kl_coef=0.001,
                             pad_token_id=0)
    loader = iter(MultiModalPromptLoader(_dataset(8), gbs, seed=0))
    seen = {}
    real_forward = worker.actor.core.hidden_states

    def spy(ids_or_h, meta, chunk=None):
        seen["image_rows"] = seen.get("image_rows", 0) + (0 if meta.image_index is None else int(meta.image_index.numel()))
        seen["mrope"] = seen.get("mrope", False) or meta.rope_table is not None
        return real_forward(ids_or_h, meta, chunk)

    worker.actor.core.hidden_states = spy
    hist = trainer.fit(loader)
    assert len(hist) == 2 and all("actor/pg_loss" in m and m["timing/rollout"] > 0 and "timing/vit_image_emb" in m for m in hist)
    assert seen["image_rows"] > 0 and seen["mrope"]            # training consumed embeddings and three-axis positions
    assert abs(hist[0]["actor/kl_loss"]) < 1e-4                # reference pass sees the same inputs as the actor
