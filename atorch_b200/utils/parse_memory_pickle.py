"""Which source files hold the device memory: reads a snapshot written by
``torch.cuda.memory._dump_snapshot`` (``_record_memory_history`` on) and sums the live allocation sizes by
the innermost frame whose file name passes the allow / block lists.
(Reference: atorch/utils/parse_memory_pickle.py:11-120.)"""
from __future__ import annotations

import argparse
import pickle
from collections import Counter
from typing import Iterable, Optional


def filename_is_allow(filename: str, whitelist: Optional[Iterable[str]]) -> bool:
    return not whitelist or any(w in filename for w in whitelist)


def parse_memory_pickle_file(pickle_file: str, blocklist: Iterable[str] = (), whitelist: Optional[Iterable[str]] = None) -> Counter:
    with open(pickle_file, "rb") as f:
        snap = pickle.load(f)
    counter: Counter = Counter()
    for seg in snap.get("segments", []):
        for blk in seg.get("blocks", []):
            if blk.get("state") != "active_allocated":
                continue
            owner = "<unknown>"
            for fr in blk.get("frames", []) or []:
                fn = fr.get("filename", "")
                if any(b in fn for b in blocklist) or not filename_is_allow(fn, whitelist):
                    continue
                owner = f"{fn}:{fr.get('line', 0)} {fr.get('name', '')}"
                break
            counter[owner] += int(blk.get("size", 0))
    return counter


def print_result(filename_counter: Counter, blocklist=(), limit: int = 20) -> None:
    total = sum(filename_counter.values())
    print(f"live device memory: {total / 2 ** 20:.1f} MiB")
    for name, size in filename_counter.most_common(limit):
        print(f"{size / 2 ** 20:10.1f} MiB  {name}")


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("pickle_file")
    ap.add_argument("--blocklist", nargs="*", default=["torch/", "site-packages"])
    ap.add_argument("--whitelist", nargs="*", default=None)
    ap.add_argument("--limit", type=int, default=20)
    return ap.parse_args(argv)


def main(argv=None) -> None:
    a = parse_args(argv)
    print_result(parse_memory_pickle_file(a.pickle_file, a.blocklist, a.whitelist), a.blocklist, a.limit)


if __name__ == "__main__":
    main()
