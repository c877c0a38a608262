"""Registry of expert classes (reference: hivemind/moe/server/layers/custom_experts.py:11-35)."""
from __future__ import annotations

import importlib.util
import os
from typing import Callable, Dict, Type

import torch
import torch.nn as nn

name_to_block: Dict[str, Type[nn.Module]] = {}
name_to_input: Dict[str, Callable[[int, int], torch.Tensor]] = {}


_loaded_files = set()


def add_custom_models_from_file(path: str) -> None:
    """Import a python file so that its ``@register_expert_class`` decorators run (once per file and process:
    servers are threads here, so several of them may name the same file)."""
    key = (os.path.abspath(path), os.path.getmtime(path))
    if key in _loaded_files:
        return
    _loaded_files.add(key)
    spec = importlib.util.spec_from_file_location("custom_module", os.path.abspath(path))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)


def register_expert_class(name: str, sample_input: Callable[[int, int], torch.Tensor]):
    """Class decorator: make an ``nn.Module`` with ``__init__(hid_dim)`` available to servers under ``name``.

    :param sample_input: ``(batch_size, hid_dim) -> example input`` (a tensor or a tuple of tensors) used to derive
      the expert's input / output schema
    """

    def _register(custom_class: Type[nn.Module]) -> Type[nn.Module]:
        if name in name_to_block or name in name_to_input:
            raise RuntimeError(f"The expert class {name} has already been registered")
        name_to_block[name] = custom_class
        name_to_input[name] = sample_input
        return custom_class

    return _register
