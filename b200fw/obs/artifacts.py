"""Run artefact files: rank 0 writes the global files, every rank its own ``*_rank{r}`` files
(src/utils/artifact_writer.py:19-88)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict


class ArtifactWriter:
    def __init__(self, output_dir: str, rank: int = 0, world_size: int = 1):
        self.output_dir, self.rank, self.world_size = output_dir, rank, world_size
        os.makedirs(output_dir, exist_ok=True)
        self._started = set()        # per-rank JSONL stems already truncated by write_rank_jsonl in this run

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    def path(self, name: str) -> str:
        return os.path.join(self.output_dir, name)

    def rank_path(self, stem: str, ext: str) -> str:
        return os.path.join(self.output_dir, f"{stem}_rank{self.rank}.{ext}")

    def write_json(self, name: str, obj: Any, all_ranks: bool = False):
        if all_ranks:
            stem, ext = os.path.splitext(name)
            path = self.rank_path(stem, ext.lstrip(".") or "json")
        elif self.is_main:
            path = self.path(name)
        else:
            return None
        with open(path, "w") as f:
            json.dump(obj, f, indent=2, default=str)
        return path

    def append_jsonl(self, stem: str, row: Dict[str, Any]):
        path = self.rank_path(stem, "jsonl")
        with open(path, "a") as f:
            f.write(json.dumps(row, default=str) + "\n")
        return path

    def write_text(self, name: str, text: str):
        if not self.is_main:
            return None
        with open(self.path(name), "w") as f:
            f.write(text)
        return self.path(name)

    # ---- the reference's method names (src/utils/artifact_writer.py:39-86) ---------------------------------
    def write_main_json(self, filename: str, data: Any):
        """Rank 0 only: ``<output_dir>/<filename>``."""
        return self.write_json(filename, data)

    def write_main_text(self, filename: str, text: str):
        return self.write_text(filename, text)

    def write_rank_json(self, base_filename: str, data: Any):
        """Every rank: ``metrics.json`` -> ``metrics_rank{r}.json``."""
        return self.write_json(base_filename, data, all_ranks=True)

    def write_rank_jsonl(self, base_filename: str, row: Dict[str, Any]):
        """Every rank: ``metrics.jsonl`` -> one appended line in ``metrics_rank{r}.jsonl``.  The first write of
        a run truncates the file, so that rows of an earlier run in the same directory do not mix in."""
        stem = os.path.splitext(base_filename)[0]
        if stem not in self._started:
            self._started.add(stem)
            open(self.rank_path(stem, "jsonl"), "w").close()
        return self.append_jsonl(stem, row)

    def close(self):
        """Files are opened per write; nothing stays open.  Kept so that callers of the reference's API work."""
        self._started.clear()

