"""mindspeed_rl_b200 — a Blackwell (sm_100a) native RL post-training framework.

The public surface mirrors what users of MindSpeed-RL rely on (``cli/train_*.py`` entry
points, the YAML configuration sections, GRPO/DAPO/PPO/DPO trainers, hybrid actor workers,
a TransferDock experience store and Megatron-mcore style checkpoints) while every layer
underneath -- training backend, paged-KV rollout engine, collectives and kernels -- lives
in this package and is written for B200.

Sub-packages
------------
config      YAML -> validated config objects
data        TransferDock / TransferQueue experience stores, packing helpers
datasets    indexed ``.bin/.idx`` datasets, templates, prompt loaders
models      GPT (dense + MoE), reward/critic head, loss registry
ops         Python front-ends of the hand-written CUDA kernels (``csrc/``)
parallel    parallel state, tensor/sequence/context/expert/pipeline parallel layers
rollout     paged-KV generation engine (scheduler, block manager, sampler)
reshard     train -> rollout weight resharding and memory offload
optim       Adam (device or pinned-host state), distributed optimizer, LR schedules
checkpoint  mcore ``torch`` format reader/writer and the HF converter
runtime     actor runtime (local multiprocessing backend, optional Ray)
workers     actor / reference / critic / reward / rule-reward workers
trainer     GRPO / DAPO / PPO / DPO driver loops
rewards     rule verifiers and math grading
tools       multi-turn tool calling
obs         metrics, loggers, profiler and tensor dump utilities
"""

__version__ = "0.1.0"
