"""TransferDock: the central experience store between the RL stages.

A table of ``prompts_num * n_samples_per_prompt`` rows and named columns of ragged 1-D
tensors.  Each column keeps a *ready* bit per row, each consumer (stage) a *consumed* bit per
row.  ``get_experience`` hands a consumer rows that are ready in all requested columns and not
yet consumed by it -- in whole prompt groups when ``get_n_samples`` -- and marks them consumed
under the consumer's lock, so stages can pull concurrently (the dock is served by a
multi-threaded actor).  Row ``i`` belongs to prompt ``i // n``; prompts are stored ``n`` times.

Partial rollout (``max_age > 1``): rows carry an ``age`` (how many policy updates behind) and a
``rollout_completed`` flag; only prompt groups whose ``n`` samples are all completed become
visible to the stages after rollout; after an update the trained rows are evicted, survivors
age by one and groups are re-ordered oldest first.

Contract and column / consumer names follow the reference
(``mindspeed_rl/trainer/utils/transfer_dock.py:28-880``); the implementation keeps all status
as vectors and samples with vectorised operations.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..utils.pad_process import padding_dict_to_tensor_dict, remove_padding_tensor_dict_to_dict
from ..utils.seqlen_balancing import get_seqlen_balanced_partitions

BASE_COLUMNS = [
    "prompts", "prompt_length", "responses", "response_length", "attention_mask", "labels",
    "input_ids", "input_ids_length", "actor_rollout", "rm_scores", "token_level_rewards",
    "old_log_prob", "ref_log_prob", "advantages", "returns",
]
BASE_CONSUMERS = [
    "trainer", "actor_rollout", "actor_image_embeds", "actor_log_prob", "ref_log_prob",
    "actor_train", "compute_advantage", "rule_reward", "reward_scores", "grpo_metrics",
]
_SEQLEN_COLUMNS = ("prompt_length", "response_length")
_BALANCED_CONSUMERS = ("ref_log_prob", "actor_log_prob", "reward_scores", "actor_train",
                       "critic_train", "critic_compute_values")


class TransferDock:
    """Column/row storage with ready bits (no consumer logic)."""

    def __init__(self, prompts_num: int, n_samples_per_prompt: int, experience_columns: Sequence[str],
                 timeout: Optional[int] = None, timeout_interval: Optional[int] = None):
        self.prompts_num = prompts_num
        self.n_samples_per_prompt = n_samples_per_prompt
        self.max_len = prompts_num * n_samples_per_prompt
        self.experience_columns = list(experience_columns)
        self.experience_data: Dict[str, List[Optional[torch.Tensor]]] = {
            c: [None] * self.max_len for c in self.experience_columns}
        self.experience_data_status: Dict[str, torch.Tensor] = {
            c: torch.zeros(self.max_len, dtype=torch.int32) for c in self.experience_columns}
        self.timeout = timeout if timeout is not None else 300
        self.timeout_interval = timeout_interval if timeout_interval is not None else 5
        self._data_lock = threading.Lock()

    def _put(self, columns: Sequence[str], experience: Sequence[Sequence[torch.Tensor]],
             indexes: Sequence[int]) -> None:
        for col, rows in zip(columns, experience):
            if col not in self.experience_data:
                raise ValueError(f"put experience: unknown column '{col}' (known: {self.experience_columns})")
            if len(rows) != len(indexes):
                raise ValueError(f"column '{col}': {len(rows)} rows for {len(indexes)} indexes")
            store, status = self.experience_data[col], self.experience_data_status[col]
            for i, idx in enumerate(indexes):
                if idx < 0:
                    continue
                if idx >= self.max_len:
                    raise ValueError(f"index {idx} out of range (max_len {self.max_len})")
                store[idx] = rows[i]
                status[idx] = 1

    def _get(self, columns: Sequence[str], indexes: Sequence[int]) -> List[List[torch.Tensor]]:
        if len(indexes) == 0:
            return [[] for _ in columns]
        if max(indexes) >= self.max_len or min(indexes) < 0:
            raise ValueError(f"indexes out of range for max_len {self.max_len}")
        out = []
        for col in columns:
            self._wait_for_data(col, indexes)
            out.append([self.experience_data[col][i] for i in indexes])
        return out

    def _wait_for_data(self, column: str, indexes: Sequence[int]) -> None:
        """Block until every requested cell is ready; complain periodically, give up after 10x."""
        idx = torch.as_tensor(list(indexes), dtype=torch.int64)
        start = time.time()
        warned = 0
        while int(self.experience_data_status[column][idx].sum()) != len(indexes):
            waited = time.time() - start
            if waited > self.timeout and waited - warned > self.timeout_interval:
                warned = waited
                print(f"[TransferDock] waiting {waited:.0f}s for column '{column}' rows {list(indexes)[:8]}...")
            if waited > 10 * self.timeout:
                raise TimeoutError(f"column '{column}' never became ready for rows {list(indexes)[:8]}")
            time.sleep(0.01)

    def _clear_experience_data_and_status(self, indexes: Optional[torch.Tensor] = None) -> None:
        if indexes is None:
            for c in self.experience_columns:
                self.experience_data[c] = [None] * self.max_len
                self.experience_data_status[c].zero_()
        else:
            for c in self.experience_columns:
                self.experience_data_status[c][indexes] = 0
                for i in indexes.tolist():
                    self.experience_data[c][i] = None

    def get_experience_data(self):
        return self.experience_data

    def get_experience_status(self):
        return self.experience_data_status

    def get_experience_len(self) -> int:
        return self.max_len


def trans_input_to_experience(data: Dict[str, Union[torch.Tensor, List[torch.Tensor]]]
                              ) -> Tuple[List[str], List[List[torch.Tensor]]]:
    """Dict of columns (2-D tensor or list of rows) -> (names, list of row lists)."""
    names, cols = [], []
    for k, v in data.items():
        names.append(k)
        if torch.is_tensor(v):
            cols.append([row for row in v] if v.dim() > 1 else [x.reshape(1) for x in v])
        else:
            cols.append(list(v))
    return names, cols


class GRPOTransferDock(TransferDock):
    def __init__(self, prompts_num: int, n_samples_per_prompt: int, metrics=None, max_age: int = 1,
                 GBS_train: int = 0, addition_columns: Optional[List[str]] = None,
                 addition_consumers: Optional[List[str]] = None, timeout: Optional[int] = None,
                 timeout_interval: Optional[int] = None):
        columns = list(BASE_COLUMNS)
        for c in addition_columns or []:
            if c not in columns:
                columns.append(c)
        super().__init__(prompts_num, n_samples_per_prompt, columns, timeout, timeout_interval)
        self.experience_consumers = list(BASE_CONSUMERS)
        for c in addition_consumers or []:
            if c not in self.experience_consumers:
                self.experience_consumers.append(c)
        self.experience_consumer_status = {c: torch.zeros(self.max_len, dtype=torch.int32)
                                           for c in self.experience_consumers}
        self.consumer_sampling_lock = {c: threading.Lock() for c in self.experience_consumers}
        self.max_age = max_age
        self.GBS_train = GBS_train
        self.rollout_completed = torch.zeros(self.max_len, dtype=torch.int32)
        self.age = torch.zeros(self.max_len, dtype=torch.int32)
        self.enable_partial_rollout = max_age > 1
        self.stop_partial_rollout_signal = False
        self.global_ready_mask = torch.zeros(self.max_len, dtype=torch.int32)
        self.max_age_all_finished = False
        if metrics is None:
            from ..obs.metrics import Metric

            metrics = Metric()
        self.metrics = metrics
        self._index_lock = threading.Lock()
        self.cur_index = 0

    # ---- metrics sink ---------------------------------------------------------------------------
    def get_metrics(self):
        return self.metrics

    def update_metrics(self, key: str = "", value=None, cumulate: bool = False) -> None:
        self.metrics.update(key, value, cumulate=cumulate)

    # ---- index hand-out (dynamic sampling fills the main dock through this) ------------------------
    def get_cur_index(self) -> int:
        return self.cur_index

    def prefetch_request_index(self, experience_num: int) -> Optional[List[int]]:
        with self._index_lock:
            if self.cur_index >= self.max_len:
                return None
            out = list(range(self.cur_index, min(self.cur_index + experience_num, self.max_len)))
            self.cur_index += experience_num
        return out

    # ---- read ------------------------------------------------------------------------------------
    def get_experience(self, consumer: str, experience_columns: List[str],
                       experience_count: Optional[int] = None, dp_size: int = 1,
                       indexes: Optional[List[int]] = None, get_n_samples: bool = True,
                       use_batch_seqlen_balance: bool = False,
                       allow_partial_ready_data: bool = False):
        """Padded batch + row indexes for ``consumer`` (``(None, None)`` when nothing is ready)."""
        if consumer not in self.experience_consumers:
            raise ValueError(f"unknown consumer '{consumer}' (known: {self.experience_consumers})")
        columns = list(experience_columns)
        want_age = "age" in columns
        if want_age:
            if not (consumer == "actor_rollout" and self.enable_partial_rollout):
                raise ValueError("column 'age' is only served to actor_rollout under partial rollout")
            columns.remove("age")
        for c in columns:
            if c not in self.experience_columns:
                raise ValueError(f"unknown column '{c}' (known: {self.experience_columns})")
        if consumer == "actor_rollout" and self.enable_partial_rollout and get_n_samples:
            raise ValueError("get_n_samples is not available for actor_rollout under partial rollout")
        if indexes is None:
            if experience_count is None or experience_count <= 0:
                raise ValueError("experience_count must be a positive integer when no indexes are given")
            if experience_count > self.max_len:
                raise ValueError(f"experience_count {experience_count} exceeds dock size {self.max_len}")
            if self.max_len % experience_count != 0 and not self.enable_partial_rollout:
                raise ValueError(f"dock size {self.max_len} must be divisible by experience_count "
                                 f"{experience_count}")
            if get_n_samples:
                if experience_count % self.n_samples_per_prompt != 0:
                    raise ValueError("experience_count must be a multiple of n_samples_per_prompt "
                                     "when get_n_samples is set")
                indexes = self._sample_ready_index_n_samples(consumer, experience_count, columns,
                                                             use_batch_seqlen_balance)
            else:
                indexes = self._sample_ready_index(consumer, experience_count, columns,
                                                   use_batch_seqlen_balance)
            if not indexes:
                return None, None
        else:
            indexes = list(indexes)
            if indexes and (max(indexes) >= self.max_len or min(indexes) < 0):
                raise ValueError(f"indexes out of range for max_len {self.max_len}")
            self.experience_consumer_status[consumer][torch.as_tensor(indexes, dtype=torch.int64)] = 1
        rows = self._get(columns, indexes)
        if consumer == "actor_rollout" and self.enable_partial_rollout:
            idx_t = torch.as_tensor(indexes, dtype=torch.int64)
            columns.append("age")
            rows.append([self.age[i].reshape(1).clone() for i in indexes])
            # responses of these rows are being regenerated / continued
            self.experience_data_status["responses"][idx_t] = 0
            self.experience_data_status["response_length"][idx_t] = 0
            n = len(indexes)
            if 0 < n < (experience_count or n):
                # pad to a multiple of dp_size with copies of the last row (index -2 = filler)
                target = -(-n // dp_size) * dp_size
                for col in rows:
                    col.extend([col[n - 1]] * (target - n))
                indexes = indexes + [-2] * (target - n)
        batch = padding_dict_to_tensor_dict(dict(zip(columns, rows)))
        return batch, indexes

    # ---- write -------------------------------------------------------------------------------------
    def put_experience(self, data_dict: Dict[str, Union[torch.Tensor, List[torch.Tensor]]],
                       indexes: Optional[List[int]] = None, is_prompt: bool = False) -> None:
        if not indexes:
            raise ValueError("put_experience needs the row indexes")
        data = remove_padding_tensor_dict_to_dict(data_dict)
        if self.enable_partial_rollout and self.GBS_train == 0:
            raise ValueError("GBS_train must be given when partial rollout is enabled")
        names, cols = trans_input_to_experience(data)
        rollout_put = "responses" in names
        if rollout_put and self.enable_partial_rollout:
            if "rollout_completed" not in names:
                raise ValueError("partial rollout: 'rollout_completed' must accompany 'responses'")
            k = names.index("rollout_completed")
            flags = cols.pop(k)
            names.pop(k)
            for i, idx in enumerate(indexes):
                if idx >= 0 and int(flags[i].reshape(-1)[0]) == 1:
                    self.rollout_completed[idx] = 1
        cols = [[self._narrow(t) for t in col] for col in cols]
        self._put(names, cols, indexes)
        idx_t = torch.as_tensor([i for i in indexes if i >= 0], dtype=torch.int64)
        if rollout_put and self.enable_partial_rollout:
            self.experience_consumer_status["actor_rollout"][idx_t] = self.rollout_completed[idx_t].clone()
        if self.enable_partial_rollout and is_prompt:
            self.experience_data_status["responses"][idx_t] = 1
            self.experience_data_status["response_length"][idx_t] = 1
            for i in idx_t.tolist():
                self.experience_data["responses"][i] = torch.tensor([-1], dtype=torch.int32)
                self.experience_data["response_length"][i] = torch.tensor([0], dtype=torch.int32)

    @staticmethod
    def _narrow(t: torch.Tensor) -> torch.Tensor:
        """Token ids and lengths travel as int32 (halves host traffic)."""
        return t.to(torch.int32) if t.dtype == torch.int64 else t

    # ---- sampling ------------------------------------------------------------------------------------
    def _ready_mask(self, columns: Sequence[str]) -> torch.Tensor:
        ready = torch.ones(self.max_len, dtype=torch.bool)
        for c in columns:
            ready &= self.experience_data_status[c] == 1
        return ready

    def _training_window(self) -> torch.Tensor:
        """Partial rollout: rows of the first ``GBS_train`` completed prompt groups.  More groups than one
        training batch may have completed when the rollout stops; every downstream stage (rewards, log-probs,
        advantages, update) must work on the same ones, so the choice is by position, not by chance."""
        n = self.n_samples_per_prompt
        done = (self.global_ready_mask.view(self.prompts_num, n).sum(dim=1) == n).nonzero(as_tuple=True)[0]
        rows = torch.zeros(self.max_len, dtype=torch.bool)
        for g in done[:self.GBS_train].tolist():
            rows[g * n:(g + 1) * n] = True
        return rows

    def _sample_ready_index(self, consumer: str, experience_count: int, columns: Sequence[str],
                            use_batch_seqlen_balance: bool = False) -> Optional[List[int]]:
        with self.consumer_sampling_lock[consumer]:
            usable = (self.experience_consumer_status[consumer] == 0) & self._ready_mask(columns)
            rollout_pr = self.enable_partial_rollout and consumer == "actor_rollout"
            if self.enable_partial_rollout and not rollout_pr:
                usable &= self._training_window()
            usable_idx = usable.nonzero(as_tuple=True)[0]
            if len(usable_idx) < experience_count:
                if rollout_pr and len(usable_idx) > 0:
                    experience_count = len(usable_idx)
                else:
                    return None
            if rollout_pr or self.enable_partial_rollout:
                picked = usable_idx[:experience_count].tolist()
            elif (use_batch_seqlen_balance and consumer in _BALANCED_CONSUMERS
                  and len(usable_idx) % experience_count == 0):
                picked = self._balanced_pick(usable_idx, experience_count, group=False)
            else:
                perm = torch.randperm(len(usable_idx))[:experience_count]
                picked = usable_idx[perm].tolist()
            if not picked:
                return None
            self.experience_consumer_status[consumer][torch.as_tensor(picked, dtype=torch.int64)] = 1
        return [int(i) for i in picked]

    def _sample_ready_index_n_samples(self, consumer: str, experience_count: int,
                                      columns: Sequence[str], use_batch_seqlen_balance: bool = False
                                      ) -> Optional[List[int]]:
        n = self.n_samples_per_prompt
        groups_wanted = experience_count // n
        with self.consumer_sampling_lock[consumer]:
            status = self.experience_consumer_status[consumer]
            free = (status.view(self.prompts_num, n) == 0).all(dim=1)
            ready = self._ready_mask(columns).view(self.prompts_num, n).all(dim=1)
            usable = free & ready
            if self.enable_partial_rollout:
                usable &= self._training_window().view(self.prompts_num, n).all(dim=1)
            usable_idx = usable.nonzero(as_tuple=True)[0]
            if len(usable_idx) < groups_wanted:
                return None
            if self.enable_partial_rollout and int(status.sum()) >= self.GBS_train * n:
                return None
            if self.enable_partial_rollout:
                groups = usable_idx[:groups_wanted].tolist()
            elif (use_batch_seqlen_balance and consumer in _BALANCED_CONSUMERS
                  and len(usable_idx) % groups_wanted == 0):
                groups = self._balanced_pick(usable_idx, groups_wanted, group=True)
            else:
                groups = usable_idx[torch.randperm(len(usable_idx))[:groups_wanted]].tolist()
            if not groups:
                return None
            rows = [g * n + j for g in groups for j in range(n)]
            status[torch.as_tensor(rows, dtype=torch.int64)] = 1
        return rows

    def _balanced_pick(self, usable_idx: torch.Tensor, count: int, group: bool) -> List[int]:
        """Split the usable rows/groups into equal parts of similar token count, take the first."""
        if len(usable_idx) == count:
            return usable_idx.tolist()
        n = self.n_samples_per_prompt

        def row_len(r: int) -> int:
            return sum(int(self.experience_data[c][r].reshape(-1)[0]) for c in _SEQLEN_COLUMNS
                       if self.experience_data[c][r] is not None)

        if group:
            lens = [sum(row_len(int(g) * n + j) for j in range(n)) for g in usable_idx]
        else:
            lens = [row_len(int(r)) for r in usable_idx]
        parts = get_seqlen_balanced_partitions(lens, len(lens) // count, equal_size=True)
        return [int(usable_idx[i]) for i in parts[0]] if parts else []

    # ---- progress ------------------------------------------------------------------------------------
    def all_consumed(self, consumer: str, get_n_samples: bool = True) -> bool:
        if self.enable_partial_rollout:
            if self.GBS_train == 0:
                raise ValueError("GBS_train must be given when partial rollout is enabled")
            if consumer == "actor_rollout":
                done, mask, _ = self.find_all_consumed_n_samples_groups("actor_rollout")
                self.stop_partial_rollout_signal = done >= self.GBS_train
                self.global_ready_mask = mask
                return done >= self.GBS_train
            return int(self.experience_consumer_status[consumer].sum()) == \
                self.GBS_train * self.n_samples_per_prompt
        return int(self.experience_consumer_status[consumer].sum()) == self.max_len

    def find_all_consumed_n_samples_groups(self, consumer: str):
        if consumer != "actor_rollout":
            raise ValueError("only actor_rollout drives the partial-rollout stop signal")
        n = self.n_samples_per_prompt
        done_groups = (self.rollout_completed.view(self.prompts_num, n) == 1).all(dim=1)
        mask = done_groups.repeat_interleave(n).to(torch.int32)
        starts = (done_groups.nonzero(as_tuple=True)[0] * n).tolist()
        return int(done_groups.sum()), mask, starts

    def get_update_ready(self, require_max_age_all_finished: bool = True) -> bool:
        done, mask, _ = self.find_all_consumed_n_samples_groups("actor_rollout")
        self.stop_partial_rollout_signal = done >= self.GBS_train
        self.global_ready_mask = mask
        if not require_max_age_all_finished:
            return self.stop_partial_rollout_signal
        oldest = self.age == self.max_age - 1
        self.max_age_all_finished = bool((self.rollout_completed[oldest] == 1).all())
        return self.stop_partial_rollout_signal and self.max_age_all_finished

    def get_incomplete_response_num(self) -> int:
        return int(self.experience_data_status["prompts"].sum() - self.rollout_completed.sum())

    def get_consumer_status(self):
        return self.experience_consumer_status

    # ---- reset -----------------------------------------------------------------------------------------
    def sort_every_n_samples_by_age(self) -> None:
        """Re-order prompt groups oldest first (stable); a group's age is the max of its rows."""
        n = self.n_samples_per_prompt
        group_age = self.age.view(self.prompts_num, n).max(dim=1).values
        self.age = group_age.repeat_interleave(n).clone()
        order = torch.argsort(group_age, descending=True, stable=True)
        rows = (order.unsqueeze(1) * n + torch.arange(n).unsqueeze(0)).reshape(-1)
        row_list = rows.tolist()
        for c in self.experience_columns:
            col = self.experience_data[c]
            self.experience_data[c] = [col[i] for i in row_list]
            self.experience_data_status[c] = self.experience_data_status[c][rows].clone()
        for c in self.experience_consumers:
            self.experience_consumer_status[c] = self.experience_consumer_status[c][rows].clone()
        self.age = self.age[rows].clone()
        self.age[self.age == -1] = 0
        self.rollout_completed = self.rollout_completed[rows].clone()
        self.global_ready_mask = self.global_ready_mask[rows].clone()

    def clear(self, consumer: str = "actor_train") -> None:
        if self.enable_partial_rollout:
            trained = (self.experience_consumer_status[consumer] == 1).nonzero(as_tuple=True)[0]
            if trained.numel() > 0:
                for c in self.experience_consumers:
                    self.experience_consumer_status[c][trained] = 0
                self._clear_experience_data_and_status(trained)
                self.age = self.age + (self.experience_data_status["input_ids"] == 1).to(torch.int32)
                self.age[trained] = -1
                self.global_ready_mask[trained] = 0
                self.rollout_completed[trained] = 0
                self.sort_every_n_samples_by_age()
            self.stop_partial_rollout_signal = False
        else:
            for c in self.experience_consumers:
                self.experience_consumer_status[c].zero_()
            self._clear_experience_data_and_status()
        self.cur_index = 0
        self.metrics.reset()


def put_prompts_experience(batch: Dict[str, List[torch.Tensor]], n_samples_per_prompt: int,
                           dataset_additional_keys: Optional[List[str]] = None,
                           indexes: Optional[List[int]] = None, add_another_batch: bool = False
                           ) -> Tuple[Dict[str, List[torch.Tensor]], List[int]]:
    """Expand a prompt batch to ``n`` rows per prompt (+ ``prompt_length`` and extra keys).

    ``add_another_batch`` offsets the default indexes by one batch (partial rollout keeps two
    batches in the dock; reference: ``transfer_dock.py:1201-1244``).
    """
    prompts = list(batch["prompts"])
    n = n_samples_per_prompt
    rows, lens = [], []
    for p in prompts:
        for _ in range(n):
            rows.append(p.reshape(-1))
            lens.append(torch.tensor([p.numel()], dtype=torch.int32))
    data: Dict[str, List[torch.Tensor]] = {"prompts": rows, "prompt_length": lens}
    for key in dataset_additional_keys or []:
        if key in batch:
            vals = []
            for v in batch[key]:
                v = v if torch.is_tensor(v) else torch.as_tensor(v)
                vals.extend([v.reshape(-1)] * n)
            data[key] = vals
    if indexes is None:
        total = len(prompts) * n
        base = total if add_another_batch else 0
        indexes = list(range(base, base + total))
    return data, indexes
