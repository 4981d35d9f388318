"""Model families by architecture name.  A family registers how to build its model from a checkpoint folder
(config.json names the architecture) and from a named random-init configuration; generate.py, bench.py and bin/trace_run
all go through here, so a new design is one `register` call away from every entry point."""
from typing import Callable, Dict, Optional

import torch

from .checkpoint import is_checkpoint_folder, read_config


class Family:
    def __init__(self, name: str, from_folder: Optional[Callable] = None, from_name: Optional[Callable] = None,
                 names: Optional[Callable] = None):
        self.name, self.from_folder, self.from_name, self.names = name, from_folder, from_name, names


_FAMILIES: Dict[str, Family] = {}


def register(family: Family) -> None:
    _FAMILIES[family.name.lower()] = family


def families():
    _load_builtin()
    return dict(_FAMILIES)


def _load_builtin():
    if _FAMILIES:
        return
    from .llama import model as _llama

    def llama_from_name(name, device, dtype):
        from .llama.generate import _random_init_model
        return _random_init_model(name, device, dtype)

    register(Family("llama", from_name=llama_from_name, names=lambda: list(_llama.transformer_configs)))
    from .bitipel import model as _bitipel
    register(Family("bitipel", from_folder=_bitipel.Bitipel.from_checkpoint, from_name=_bitipel.Bitipel.from_name,
                    names=lambda: list(_bitipel.bitipel_configs)))
    from .tadolix import model as _tadolix
    register(Family("tadolix", from_folder=_tadolix.Tadolix.from_checkpoint, from_name=_tadolix.Tadolix.from_name,
                    names=lambda: list(_tadolix.tadolix_configs)))
    from .rutusun import model as _rutusun
    register(Family("rutusun", from_folder=_rutusun.Rutusun.from_checkpoint, from_name=_rutusun.Rutusun.from_name,
                    names=lambda: list(_rutusun.rutusun_configs)))
    from .fedipel import model as _fedipel
    register(Family("fedipel", from_folder=_fedipel.Fedipel.from_checkpoint, from_name=_fedipel.Fedipel.from_name,
                    names=lambda: list(_fedipel.fedipel_configs)))


def architecture_of(folder) -> str:
    cfg = read_config(folder)
    arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0] or cfg.get("model_type")
    if not arch:
        raise ValueError(f"{folder}/config.json names no architecture")
    return str(arch)


def load_checkpoint_folder(folder, device="cuda", dtype=torch.bfloat16):
    """The model whose architecture the folder's config.json names, with the folder's weights, on `device` in `dtype`."""
    _load_builtin()
    assert is_checkpoint_folder(folder), f"{folder}: expected config.json and model.safetensors"
    arch = architecture_of(folder)
    fam = _FAMILIES.get(arch.lower())
    if fam is None or fam.from_folder is None:
        raise KeyError(f"no model family registered for architecture {arch!r} (have: {sorted(_FAMILIES)})")
    return fam.from_folder(folder, device=device, dtype=dtype)


def random_init(name: str, device="cuda", dtype=torch.bfloat16):
    """A named configuration with seeded random weights; the family is found by the names it lists."""
    _load_builtin()
    for fam in _FAMILIES.values():
        if fam.from_name is not None and fam.names is not None and name in fam.names():
            return fam.from_name(name, device, dtype)
    return _FAMILIES["llama"].from_name(name, device, dtype)   # the Llama family also matches names by substring
