"""Vision-encoder worker: computes the image embeddings of every prompt once per iteration.

Stage ``compute_image_embeds`` (reference: ``mindspeed_rl/workers/vit_worker.py:100-189``, consumer
``actor_image_embeds``): pull prompt indexes from the experience store, read the prompts'
``pixel_values`` / ``image_grid_thw`` from the multimodal store, run the vision tower, write
``vit_embeds`` back (one block of rows per prompt).  The rollout, log-prob and update stages then
read the embeddings instead of running the tower again (``reuse_image_embeds``).  The worker can
live on the actor's ranks (``colocate_actor_and_vit``) or on a rank range of its own
(``vit_resource``); the tower is replicated on its ranks and prompts are dealt out data-parallel.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..data.mm_transfer_dock import unpack_mm_experience
from ..models.vit import VisionConfig, VisionTower
from .base_worker import BaseWorker, profiled_stage


class VitWorker(BaseWorker):
    def __init__(self, vit_config, rl_config, llm_hidden_size: int, td=None, mm_td=None, *, device=None,
                 seed: int = 1234, vision_config: Optional[VisionConfig] = None):
        super().__init__(td, 0)
        self.mm_td = mm_td
        self.megatron_config, self.rl_config = vit_config, rl_config
        self.vision_config = vision_config or VisionConfig.from_megatron(vit_config, llm_hidden_size)
        self.device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.seed = seed
        self.tower: Optional[VisionTower] = None
        self.iteration = 0

    def initialize(self) -> None:
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.tower = VisionTower(self.vision_config, self.device, dtype, self.seed).eval()
        for p in self.tower.parameters():
            p.requires_grad_(False)
        load = getattr(self.megatron_config, "load", None)
        if load:
            state = torch.load(load, map_location="cpu", weights_only=True)
            self.tower.load_state_dict(state.get("model", state))

    def init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None) -> None:
        self.td, self.mm_td = td, mm_td if mm_td is not None else self.mm_td

    def get_iteration(self) -> int:
        return self.iteration

    def get_consumed_train_samples(self) -> int:
        return 0

    def save_checkpoint(self, iteration: int) -> None:
        pass                                            # frozen

    @profiled_stage("vit_compute_image_embeds")
    def compute_image_embeds(self) -> None:
        rl = self.rl_config
        n = rl.n_samples_per_prompt
        count = getattr(rl, "actor_image_embeds_dispatch_size", None) or n
        start = time.time()
        while True:
            batch, idx, finished = self.dispatch_transfer_dock_data("actor_image_embeds", ["prompts", "prompt_length"],
                                                                    count, get_n_samples=True)
            if finished:
                break
            if batch is None:
                time.sleep(0.002)
                continue
            prompts = sorted({i // n for i in idx if i >= 0})
            media = self.mm_td.get_experience("actor_image_embeds", ["pixel_values", "image_grid_thw", "image_num",
                                                                     "video_num"], [p * n for p in prompts],
                                              get_n_samples=False)
            if media and media.get("pixel_values") is not None and media["pixel_values"].numel():
                embeds = self.tower(media["pixel_values"], media["image_grid_thw"]).float().cpu()
                per_prompt = unpack_mm_experience(dict(vit_embeds=embeds, image_grid_thw=media["image_grid_thw"],
                                                       image_num=media["image_num"], video_num=media["video_num"]),
                                                  merge_size=self.vision_config.spatial_merge_size)
                if self.is_writer():
                    self.mm_td.put_experience({"vit_embeds": per_prompt["vit_embeds"]}, prompts)
        self.update_metrics("timing/vit_image_emb", [round(time.time(), 4), round(start, 4)])
        self.iteration += 1
