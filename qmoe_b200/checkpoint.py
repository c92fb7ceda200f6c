"""Compressed-checkpoint directory in the reference's on-disk format (sub1.py:170-214, read back at
sub1.py:250,284-292), without the HuggingFace model surgery around it.

Directory layout (unchanged, so published ``*_qmoe`` checkpoints load as they are):

* ``config.json``   the model config (written verbatim from a dict here)
* ``noexp.pt``      state dict of all non-expert parameters, bf16
* ``exp%02d.pt``    one file per sparse layer in processing order; keys
                    ``<layer>.mlp.experts.expert_<j>.<wi|wo>.<w_comp|row_off|ter_minmax|weight>``
                    (switch.py:424-427, sub1.py:196-204), CPU tensors
* ``sizes.pt``      ``'<layer>.mlp.experts.expert_<j>.<wi|wo>' -> w_comp.numel()``

:class:`Sub1CheckpointWriter` mirrors ``Sub1CheckpointManager`` (add_expert / save_experts / finalize);
:func:`load_expert_store` builds the flat :class:`~qmoe_b200.sub1.ExpertStore` of one sparse layer
for a slice of its experts, which is what an expert-parallel rank needs.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .sub1 import ExpertStore, Sub1Linear

_SKIP = {"sizes.pt", "config.json", "README.md", ".gitattributes", ".git", "noexp.pt"}
_EXPERT_KEY = re.compile(r"^(?P<layer>.+\.mlp)\.experts\.expert_(?P<j>\d+)\.(?P<which>wi|wo)\.(?P<buf>\w+)$")


def expert_name(layer: str, j: int) -> str:
    """``<layer>.experts.expert_<j>`` with ``layer`` such as ``encoder.block.1.layer.1.mlp``."""
    return f"{layer}.experts.expert_{j}"


class Sub1CheckpointWriter:
    """Writes a compressed checkpoint directory (``Sub1CheckpointManager``, sub1.py:170-214)."""

    def __init__(self, path: str, config: Optional[dict] = None, nonexpert_state: Optional[Dict[str, torch.Tensor]] = None):
        os.makedirs(path, exist_ok=True)
        self.path = path
        if config is not None:
            cfg = dict(config)
            cfg["torch_dtype"] = "bfloat16"                       # sub1.py:186-187
            with open(os.path.join(path, "config.json"), "w") as f:
                json.dump(cfg, f, indent=2)
        if nonexpert_state is not None:                           # sub1.py:174-189
            torch.save({k: (v.bfloat16() if v.is_floating_point() else v).cpu() for k, v in nonexpert_state.items()},
                       os.path.join(path, "noexp.pt"))
        self.sd_exp: List[Optional[dict]] = [{}]
        self.sizes: Dict[str, int] = {}

    def add_packed(self, name: str, wi: Sub1Linear, wo: Sub1Linear) -> None:
        """Add one already compressed expert under ``name`` (see :func:`expert_name`)."""
        for which, lin in (("wi", wi), ("wo", wo)):
            for n, p in lin.state_dict().items():
                self.sd_exp[-1][f"{name}.{which}.{n}"] = p.cpu()
            self.sizes[f"{name}.{which}"] = lin.w_comp.numel()

    def add_expert(self, name: str, wi_weight: torch.Tensor, wo_weight: torch.Tensor) -> None:
        """Compress the ternary matrices of one expert on their device and add them
        (``add_expert``, sub1.py:196-204)."""
        self.add_packed(name, Sub1Linear.make(wi_weight), Sub1Linear.make(wo_weight))

    def save_experts(self) -> str:
        """Write the experts added since the last call as the next ``exp%02d.pt`` (sub1.py:207-210)."""
        fn = os.path.join(self.path, "exp%02d.pt" % (len(self.sd_exp) - 1))
        torch.save(self.sd_exp[-1], fn)
        self.sd_exp[-1] = None
        self.sd_exp.append({})
        return fn

    def finalize(self) -> None:
        torch.save(self.sizes, os.path.join(self.path, "sizes.pt"))  # sub1.py:213-214


def expert_files(path: str) -> List[str]:
    """The per-layer expert files of a checkpoint directory, in processing order; like the
    reference's loader every file is an expert file unless it is one of the known others
    (sub1.py:285-292)."""
    return sorted(f for f in os.listdir(path) if f not in _SKIP and f.endswith(".pt"))


def read_sizes(path: str) -> Dict[str, int]:
    return torch.load(os.path.join(path, "sizes.pt"))


def read_config(path: str) -> dict:
    """``config.json`` of a checkpoint directory (the model configuration, sub1.py:232)."""
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def read_nonexpert(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    """``noexp.pt``: the state dict of every non-expert parameter (router classifiers, attention,
    embeddings), bf16, as the reference copies it into its model (sub1.py:284-292)."""
    return torch.load(os.path.join(path, "noexp.pt"), map_location=torch.device(device))


def layers_of_file(state: Dict[str, torch.Tensor]) -> Dict[str, List[int]]:
    """``{layer prefix: sorted expert indices}`` found in one expert file."""
    found: Dict[str, set] = {}
    for k in state:
        m = _EXPERT_KEY.match(k)
        if m:
            found.setdefault(m.group("layer"), set()).add(int(m.group("j")))
    return {layer: sorted(js) for layer, js in found.items()}


def load_expert_store(path: str, file_name: str, experts: Optional[Iterable[int]] = None,
                      device="cpu", layer: Optional[str] = None) -> Tuple[ExpertStore, str, List[int]]:
    """Read one ``expNN.pt`` and build the :class:`ExpertStore` of the given expert indices (default:
    all) on ``device``.  Returns (store, layer prefix, expert indices); local expert ``i`` of the
    store is ``indices[i]``.  Matrix shapes come from the buffers themselves: height =
    ``row_off.numel() - 1``; wi is ``[d_ff, d_model]`` and wo ``[d_model, d_ff]``."""
    state = torch.load(os.path.join(path, file_name), map_location="cpu")
    layers = layers_of_file(state)
    if layer is None:
        if len(layers) != 1:
            raise ValueError(f"{file_name} holds {len(layers)} sparse layers; name one of {sorted(layers)}")
        layer = next(iter(layers))
    have = layers[layer]
    idx = have if experts is None else [int(j) for j in experts]
    missing = [j for j in idx if j not in have]
    if missing:
        raise KeyError(f"experts {missing} are not in {file_name}")
    sizes = read_sizes(path) if os.path.exists(os.path.join(path, "sizes.pt")) else {}
    dev = torch.device(device)
    parts = []
    d_ff = d_model = None
    for j in idx:
        name = expert_name(layer, j)
        wi_h = state[f"{name}.wi.row_off"].numel() - 1
        wo_h = state[f"{name}.wo.row_off"].numel() - 1
        d_ff, d_model = wi_h, wo_h
        for which, h, w in (("wi", wi_h, wo_h), ("wo", wo_h, wi_h)):
            w_comp = state[f"{name}.{which}.w_comp"]
            if sizes and sizes.get(f"{name}.{which}", w_comp.numel()) != w_comp.numel():
                raise ValueError(f"sizes.pt disagrees with {name}.{which}.w_comp")
            parts.append((w_comp.to(dev), state[f"{name}.{which}.row_off"].to(dev),
                          state[f"{name}.{which}.ter_minmax"].to(dev), h, w))
    return ExpertStore.from_matrices(parts, d_model, d_ff), layer, idx


def load_linear(state: Dict[str, torch.Tensor], prefix: str, device="cpu") -> Sub1Linear:
    """One :class:`Sub1Linear` from the four buffers under ``prefix`` (``...expert_<j>.wi``)."""
    lin = Sub1Linear(state[f"{prefix}.row_off"].numel() - 1, state[f"{prefix}.w_comp"].numel())
    lin.load_state_dict({k: state[f"{prefix}.{k}"] for k in ("w_comp", "row_off", "ter_minmax", "weight")})
    return lin.to(device)
