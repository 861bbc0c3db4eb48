"""Multimodal per-prompt store: lookups by sample index, consumer column sets, merge / unpack round trip."""
import torch

from mindspeed_rl_b200.data.mm_transfer_dock import MMGRPOTransferDock, merge_mm_columns, unpack_mm_experience


def _prompt(n_images, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = torch.tensor([[3, 4 + i, 6] for i in range(n_images)])
    images = [torch.rand(*s.tolist(), generator=g) for s in shapes]
    grid = torch.tensor([[1, 2 + i, 4] for i in range(n_images)])            # t, h, w patches
    pixel = torch.cat([torch.rand(int(gr.prod()), 8, generator=g) for gr in grid])
    return dict(image=torch.cat([im.reshape(1, -1) for im in images], dim=1), image_shape=shapes,
                image_num=n_images, video=torch.zeros(1, 0), video_shape=torch.zeros(0, 4, dtype=torch.long),
                video_fps=[], video_num=0, pixel_values=pixel, image_grid_thw=grid, labels=f"answer-{seed}"), images


def test_store_lookup_merge_and_unpack():
    n = 4
    dock = MMGRPOTransferDock(prompts_num=3, n_samples_per_prompt=n)
    assert dock.get_columns("actor_train") == []                      # nothing stored yet: text-only behaviour
    prompts, originals = zip(*[_prompt(k, 10 + k) for k in (2, 1, 3)])
    batch = {c: [p[c] for p in prompts] for c in prompts[0]}
    dock.put_experience(batch, [0, 1, 2])
    assert dock.get_columns("actor_train") == ["pixel_values", "image_grid_thw", "image_num", "video_num"]
    assert dock.get_columns("unknown") == []
    # sample indexes 8..11 are the 4 samples of prompt 2, 0..3 of prompt 0
    idx = list(range(8, 12)) + list(range(0, 4))
    got = dock.get_experience("actor_train", dock.get_columns("actor_train"), idx)
    assert got["image_num"].reshape(-1).tolist() == [3, 2]
    assert got["pixel_values"].shape[0] == prompts[2]["pixel_values"].shape[0] + prompts[0]["pixel_values"].shape[0]
    un = unpack_mm_experience(got)
    assert torch.equal(un["pixel_values"][0], prompts[2]["pixel_values"])
    assert torch.equal(un["pixel_values"][1], prompts[0]["pixel_values"])
    assert [g.shape[0] for g in un["image_grid_thw"]] == [3, 2]
    # raw media for the rollout: images come back with their shapes, grouped per prompt
    roll = dock.get_experience("actor_rollout", dock.get_columns("actor_rollout"), idx)
    un = unpack_mm_experience(roll)
    assert [len(g) for g in un["image"]] == [3, 2]
    for a, b in zip(un["image"][0], originals[2]):
        assert torch.equal(a, b)
    # one sample index per prompt when get_n_samples is off
    lab = dock.get_experience("rule_reward", ["labels"], [5, 9], get_n_samples=False)
    assert lab["labels"] == ["answer-11", "answer-13"]
    dock.clear()
    assert dock.get_columns("rule_reward") == []


def test_reuse_image_embeds_changes_the_readers():
    dock = MMGRPOTransferDock(2, 2, reuse_image_embeds=True)
    assert dock.consumer_columns["actor_image_embeds"][0] == "pixel_values"
    assert dock.consumer_columns["actor_train"][0] == "vit_embeds"
    grid = torch.tensor([[1, 4, 4], [1, 2, 2]])
    emb = torch.arange((16 + 4) // 4 * 3, dtype=torch.float32).reshape(-1, 3)          # after a 2x2 spatial merge
    merged = merge_mm_columns(dict(vit_embeds=[emb], image_grid_thw=[grid], image_num=[2], video_num=[0]))
    un = unpack_mm_experience(merged, merge_size=2)
    assert un["vit_embeds"][0].shape == (5, 3) and torch.equal(un["vit_embeds"][0], emb)


def test_mrope_positions_for_text_image_text():
    from mindspeed_rl_b200.datasets.mm_utils import get_rope_index
    IMG, START = 9, 8
    # 2 text tokens, vision start, a 1 x 4 x 6 image (merge 2 -> 2 x 3 = 6 placeholders), 3 text tokens, 2 pads
    ids = torch.tensor([[5, 6, START] + [IMG] * 6 + [7, 7, 7] + [0, 0]])
    mask = torch.tensor([[1] * 12 + [0, 0]])
    pos, delta = get_rope_index(ids, torch.tensor([[1, 4, 6]]), None, mask, spatial_merge_size=2,
                                image_token_id=IMG, vision_start_token_id=START)
    t, h, w = pos[0, 0].tolist(), pos[1, 0].tolist(), pos[2, 0].tolist()
    assert t[:3] == h[:3] == w[:3] == [0, 1, 2]
    assert t[3:9] == [3] * 6                       # one temporal slice
    assert h[3:9] == [3, 3, 3, 4, 4, 4] and w[3:9] == [3, 4, 5, 3, 4, 5]
    assert t[9:12] == h[9:12] == w[9:12] == [6, 7, 8]      # continues after the largest index used (5) + 1
    assert t[12:] == [1, 1]                         # padding
    assert delta.tolist() == [[9 - 14]]
    # text only: plain positions
    pos, delta = get_rope_index(torch.tensor([[4, 4, 4, 0]]), attention_mask=torch.tensor([[1, 1, 1, 0]]))
    assert pos[:, 0].tolist() == [[0, 1, 2, 1]] * 3 and delta.tolist() == [[3 - 4]]
