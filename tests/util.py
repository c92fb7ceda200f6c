"""Helpers shared by the GPU parity tests: seeded matrices encoded by the CPU oracle."""
import numpy as np
import torch

from oracle import oracle as O
from qmoe_b200 import synth


class Matrix:
    """One synthetic compressed matrix: CPU truth (symbols, oracle codes) + device tensors."""

    def __init__(self, height, width, seed=0, matrix_id=0, p_zero=0.9, sym=None, minmax=None, device=None):
        dec, trie = O.build_dictionary()
        if sym is None:
            sym, mm = synth.matrix_cpu(height, width, seed, matrix_id, p_zero)
        else:
            mm = synth.row_scales(height, seed, matrix_id)
        if minmax is not None:
            mm = minmax
        self.height, self.width = height, width
        self.sym = np.ascontiguousarray(sym, dtype=np.uint8)
        self.codes, self.row_off = O.encode_matrix(trie, self.sym)
        self.minmax = mm                                   # bf16 torch tensor [2H]
        self.minmax_bits = mm.view(torch.int16).numpy().view(np.uint16)
        if device is not None:
            self.to(device)

    def to(self, device):
        self.d_codes = torch.from_numpy(self.codes.view(np.int16)).to(device)
        self.d_row_off = torch.from_numpy(self.row_off).to(device)
        self.d_minmax = self.minmax.to(device)
        return self

    def dense(self):
        """fp32 [H, W] decoded weights {0, min_r, max_r}."""
        mm = self.minmax.float().numpy().reshape(-1, 2)
        deq = np.concatenate([np.zeros((self.height, 1), np.float32), mm], 1)
        return np.take_along_axis(deq, self.sym.astype(np.int64), 1)

    def oracle_matvec(self, x_bf16: torch.Tensor, y0_bf16: torch.Tensor = None):
        """Oracle y (bf16 torch [t, H]) for x [t, W]; y0 is the accumulate-into value (default 0)."""
        dec, _ = O.build_dictionary()
        x_bits = x_bf16.reshape(-1, self.width).contiguous().view(torch.int16).numpy().view(np.uint16)
        t = x_bits.shape[0]
        if y0_bf16 is None:
            y_bits = np.zeros((t, self.height), dtype=np.uint16)
        else:
            y_bits = y0_bf16.reshape(t, self.height).contiguous().view(torch.int16).numpy().view(np.uint16).copy()
        O.matvec(dec, self.codes, self.row_off, self.minmax_bits, x_bits, y_bits, self.height, self.width)
        return torch.from_numpy(y_bits.view(np.int16)).view(torch.bfloat16)


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref| -- the error measure of the 1e-2 layer-parity bound."""
    got, ref = got.float().cpu(), ref.float().cpu()
    return float((got - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


def randn_bf16(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()


class Expert:
    """wi [d_ff, d_model] and wo [d_model, d_ff] of one synthetic expert."""

    def __init__(self, d_model, d_ff, seed, expert_id, p_zero=0.9):
        self.wi = Matrix(d_ff, d_model, seed, 2 * expert_id, p_zero)
        self.wo = Matrix(d_model, d_ff, seed, 2 * expert_id + 1, p_zero)
        self.d_model, self.d_ff = d_model, d_ff

    def oracle_ffn(self, x_bf16: torch.Tensor) -> torch.Tensor:
        dec, _ = O.build_dictionary()
        x_bits = x_bf16.reshape(-1, self.d_model).contiguous().view(torch.int16).numpy().view(np.uint16)
        y = O.expert_ffn(dec, (self.wi.codes, self.wi.row_off, self.wi.minmax_bits),
                         (self.wo.codes, self.wo.row_off, self.wo.minmax_bits), x_bits, self.d_model, self.d_ff)
        return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)


def store_from_experts(experts, device):
    from qmoe_b200.sub1 import ExpertStore
    parts = []
    for e in experts:
        for m in (e.wi, e.wo):
            m.to(device)
            parts.append((m.d_codes, m.d_row_off, m.d_minmax, m.height, m.width))
    return ExpertStore.from_matrices(parts, experts[0].d_model, experts[0].d_ff)


def reference_router(logits: torch.Tensor, capacity: int):
    """The Switch top-1 router of transformers 4.28 as the reference uses it (sub1.py:310):
    returns (one-hot mask after the capacity rule [B, S, E], router_probs bf16 [B, S, 1])."""
    probs = torch.softmax(logits.float(), dim=-1, dtype=torch.float32).to(torch.bfloat16)
    index = torch.argmax(probs, dim=-1)
    one_hot = torch.nn.functional.one_hot(index, num_classes=logits.shape[-1])
    priority = torch.cumsum(one_hot, dim=-2)
    one_hot = one_hot * (priority <= capacity)
    return one_hot, torch.max(probs, dim=-1).values.unsqueeze(-1)


def reference_moe(hidden: torch.Tensor, logits: torch.Tensor, experts, capacity: int) -> torch.Tensor:
    """FasterMLP.forward (sub1.py:306-321) on the CPU with the oracle as the expert FFN."""
    mask, probs = reference_router(logits, capacity)
    nxt = hidden.clone()
    for idx in torch.nonzero(mask.sum(dim=(0, 1)), as_tuple=True)[0].tolist():
        tok = mask[:, :, idx].bool()
        nxt[tok] = experts[idx].oracle_ffn(hidden[tok])
    return probs * nxt
