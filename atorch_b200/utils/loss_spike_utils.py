"""``TokenLossSpike``: record training-loss spikes to a file for later inspection.

``save_loss(file_name, cur_loss, cur_iter, losses_str, sample_infos_str)`` appends one tab-separated
line ``time  iter  loss  losses  sample_infos`` when ``cur_loss > min_loss`` and ``cur_iter >= min_iter``;
``decode_loss_spike`` parses such files and, given a ``sample_infos -> text`` decoder, reconstructs
the offending samples. (Reference: atorch/utils/loss_spike_utils.py:13-156.)
"""
from __future__ import annotations

import datetime
import os
from typing import Callable, List, Optional


class LossSpikeBase:
    def __init__(self, loss_spike_save_dir: str, sample_data_paths=None, each_sample_len: int = 0,
                 min_iter: int = 0, min_loss: float = 4.0, loss_info_splitter: str = "\t",
                 loss_sample_str_splitter: str = ","):
        self.loss_spike_save_dir = loss_spike_save_dir
        self.sample_data_paths, self.each_sample_len = sample_data_paths, each_sample_len
        self.min_iter, self.min_loss = min_iter, min_loss
        self.loss_info_splitter, self.loss_sample_str_splitter = loss_info_splitter, loss_sample_str_splitter
        os.makedirs(loss_spike_save_dir, exist_ok=True)


class TokenLossSpike(LossSpikeBase):
    def save_loss(self, file_name: str, cur_loss: float, cur_iter: int, *args, **kwargs) -> bool:
        losses_str, sample_infos_str = kwargs.get("losses_str", args[0] if args else ""), \
            kwargs.get("sample_infos_str", args[1] if len(args) > 1 else "")
        if cur_loss > self.min_loss and cur_iter >= self.min_iter:
            now = datetime.datetime.now().strftime("%Y-%m-%d %H:%M:%S")
            line = self.loss_info_splitter.join([now, str(cur_iter), str(cur_loss), losses_str, sample_infos_str])
            with open(os.path.join(self.loss_spike_save_dir, file_name), "a") as f:
                f.write(line + "\n")
            return True
        return False

    def parse(self, file_name: str) -> List[dict]:
        out = []
        with open(os.path.join(self.loss_spike_save_dir, file_name)) as f:
            for line in f:
                parts = line.rstrip("\n").split(self.loss_info_splitter)
                if len(parts) < 5:
                    continue
                out.append({"time": parts[0], "iter": int(parts[1]), "loss": float(parts[2]),
                            "losses": [float(x) for x in parts[3].split(self.loss_sample_str_splitter) if x],
                            "sample_infos": [x for x in parts[4].split(self.loss_sample_str_splitter) if x]})
        return out

    def decode_loss_spike(self, result_file_path: str, tokenizer=None, min_iter: Optional[int] = None,
                          min_loss: Optional[float] = None, fetch_sample: Optional[Callable] = None) -> int:
        """Write decoded samples of all recorded spikes (filtered) into ``result_file_path``; returns the count."""
        n = 0
        with open(result_file_path, "w") as out:
            for fn in sorted(os.listdir(self.loss_spike_save_dir)):
                for rec in self.parse(fn):
                    if (min_iter is not None and rec["iter"] < min_iter) or \
                            (min_loss is not None and rec["loss"] < min_loss):
                        continue
                    for info in rec["sample_infos"]:
                        ids = fetch_sample(info) if fetch_sample is not None else None
                        text = tokenizer.decode(ids) if (tokenizer is not None and ids is not None) else str(ids)
                        out.write(f"{rec['iter']}\t{rec['loss']}\t{info}\t{text}\n")
                        n += 1
        return n
