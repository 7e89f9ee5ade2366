"""Ready-made programs: bytecode streams recorded from the gint frontend / conductor, wrapped as executables.

``gint_b200/data/programs.json`` holds int32 bytecode streams and tensor descriptors that were produced by running
the reference's own frontend, small-matrix programs and torch.compile backend (see ``tests/golden/make_golden.py``).
``RecordedProgram`` turns one record into a ``BaseExecutableProgram`` so it runs through the normal executor path,
exactly as the conductor's compiled subgraphs do (``gint/conductor/compiler.py:300-328``).
"""
from __future__ import annotations

import json
import os
from functools import lru_cache
from typing import Optional

import numpy

from .host.executor import BaseExecutableProgram, ProgramData, ProgramTensorInfo

DEFAULT_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "programs.json")


@lru_cache(maxsize=4)
def load_records(path: Optional[str] = None) -> dict:
    with open(path or DEFAULT_GOLDEN) as f:
        return json.load(f)


class RecordedProgram(BaseExecutableProgram):
    """A fixed bytecode stream + descriptors; one cache entry, like a conductor subgraph."""

    def __init__(self, record: dict, name: str = "") -> None:
        super().__init__()
        self.name = name
        self.bytecode = numpy.asarray(record["bytecode"], dtype=numpy.int32)
        self.tensor_infos = [ProgramTensorInfo(**{k: list(v) if isinstance(v, list) else v for k, v in t.items()})
                             for t in record["infos"]]
        self.input_indices = list(record.get("input_indices") or range(len(self.tensor_infos)))
        self.grid_dim = int(record["grid_dim"])
        self.arg_roles = list(record.get("arg_roles", []))

    def get_program(self, *args, **extra_kwargs) -> ProgramData:
        return ProgramData(self.bytecode, self.tensor_infos, list(self.input_indices))

    def cache_policy(self, *args, **extra_kwargs):
        return None

    @property
    def n_instructions(self) -> int:
        return len(self.bytecode) // 2


def recorded(name: str, path: Optional[str] = None) -> RecordedProgram:
    return RecordedProgram(load_records(path)[name], name)
