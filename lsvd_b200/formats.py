"""Readers of the reference's on-disk formats for the hybrid FFN, producing real int8 buffers.

  * the channel-group JSON written by the analysis pass and read back by ``load_channel_groups``
    (fake_quant/utils/hybrid_ffn_utils.py:2774-2823): ``{"layers": {"<idx>": {"svd_idx", "quant_idx", "perm", "n_svd",
    "svd_rank", "d_ffn", "d_in", "greedy_accept_order"?}}, ...}``;
  * the quantised-model checkpoint written with ``--save_qmodel_path``
    (fake_quant/main_llava_next_hybrid_ffn.py:365-375): ``torch.save({"model": state_dict, "w_quantizers": {...}})``, the
    weights being fake-quantised fp16 (integer code times per-row scale) and ``w_quantizers`` mapping
    ``model.layers.<i>.<target>`` (targets of fake_quant/utils/hybrid_ffn_utils.py:2870-2883) to the reference's
    ``WeightQuantizer`` objects that hold the scales.

Host code only: it runs once, offline, before the first forward pass.
"""
from __future__ import annotations

import io
import json
import pickle
from typing import Dict, List, Optional, Tuple

import torch


# ------------------------------------------------------------------------------------------ channel groups
def load_channel_groups(path: str) -> dict:
    """The groups dict with its integer fields restored, as the reference's loader returns it
    (fake_quant/utils/hybrid_ffn_utils.py:2807-2823).  Raises ``KeyError`` / ``ValueError`` on a malformed file."""
    with open(path, "r") as f:
        groups = json.load(f)
    if "layers" not in groups:
        raise KeyError("channel-group file without a 'layers' table: %s" % path)
    for info in groups["layers"].values():
        for key in ("svd_idx", "quant_idx", "perm"):
            info[key] = [int(v) for v in info[key]]
        info["n_svd"] = int(info["n_svd"])
        info["svd_rank"] = int(info["svd_rank"])
        if "greedy_accept_order" in info:
            info["greedy_accept_order"] = [int(v) for v in info["greedy_accept_order"]]
    return groups


def resolve_channel_group(group: dict, d_ffn: int, n_svd: Optional[int] = None) -> Tuple[List[int], List[int], List[int], Optional[int]]:
    """(svd_idx, quant_idx, perm, rank) for one layer of a loaded file.

    With ``n_svd`` different from the stored count and a stored ``greedy_accept_order`` the groups are re-derived the way
    the reference does for another SVD ratio (fake_quant/utils/hybrid_ffn_utils.py:1123-1148): the first
    ``d_ffn - n_svd`` accepted channels go to the RTN group, padded with never-accepted channels in index order; the SVD
    group is every other channel in index order; ``perm = svd_idx + quant_idx``; the rank is then left to the caller
    (``None``).  Otherwise the stored lists and rank are returned (``:1149-1154``)."""
    stored = int(group.get("n_svd", len(group["svd_idx"])))
    if n_svd is not None and n_svd != stored and "greedy_accept_order" in group:
        order = list(group["greedy_accept_order"])
        n_quant = d_ffn - n_svd
        if n_quant <= len(order):
            quant_idx = order[:n_quant]
        else:
            seen = set(order)
            extra = [c for c in range(d_ffn) if c not in seen]
            quant_idx = order + extra[:n_quant - len(order)]
        qset = set(quant_idx)
        svd_idx = [c for c in range(d_ffn) if c not in qset]
        return svd_idx, quant_idx, svd_idx + quant_idx, None
    svd_idx, quant_idx, perm = list(group["svd_idx"]), list(group["quant_idx"]), list(group["perm"])
    if sorted(perm) != list(range(d_ffn)):
        raise ValueError("perm of the channel group is not a permutation of 0..d_ffn-1")
    if perm != svd_idx + quant_idx:
        raise ValueError("perm of the channel group is not [svd_idx | quant_idx]")
    return svd_idx, quant_idx, perm, int(group["svd_rank"])


# ------------------------------------------------------------------------------------------ checkpoints
class _Opaque:
    """Stand-in for a pickled object whose class is not importable here (the reference's quantiser classes): keeps
    the attribute dict."""

    def __init__(self, *a, **k):
        pass

    def __setstate__(self, state):
        if isinstance(state, dict):
            self.__dict__.update(state)
        else:
            self.__dict__["_state"] = state


class _TolerantUnpickler(pickle.Unpickler):
    def find_class(self, module, name):
        try:
            return super().find_class(module, name)
        except (ImportError, AttributeError):
            return type(name, (_Opaque,), {"__module__": module})


class _tolerant_pickle:
    """The ``pickle_module`` interface ``torch.load`` expects, with the tolerant unpickler."""
    __name__ = "pickle"
    Unpickler = _TolerantUnpickler
    load = staticmethod(lambda f, **kw: _TolerantUnpickler(f, **kw).load())
    loads = staticmethod(lambda b, **kw: _TolerantUnpickler(io.BytesIO(b), **kw).load())


def _quantizer_scale(qz) -> Optional[torch.Tensor]:
    """The per-row scale ``[out]`` fp32 held by a weight quantiser (a module with a ``scale`` buffer, its stand-in, a
    dict, or a tensor)."""
    if qz is None:
        return None
    if isinstance(qz, torch.Tensor):
        s = qz
    elif isinstance(qz, dict):
        s = qz.get("scale")
    else:
        d = getattr(qz, "__dict__", {})
        s = d.get("scale")
        if s is None and isinstance(d.get("_buffers"), dict):
            s = d["_buffers"].get("scale")
        if s is None:
            s = getattr(qz, "scale", None)
    return None if s is None else s.detach().float().flatten().cpu()


def load_qmodel(path: str) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    """(state dict, {target name: per-row scales fp32}) of a ``--save_qmodel_path`` checkpoint.  The quantiser objects are
    read without the reference's classes being importable.  The file is a pickle (the reference writes it with a plain
    ``torch.save`` of Python objects): like ``torch.load(weights_only=False)`` this executes what the file says, so load
    only checkpoints you made or trust."""
    blob = torch.load(path, map_location="cpu", weights_only=False, pickle_module=_tolerant_pickle)
    if "model" not in blob:
        raise KeyError("checkpoint without a 'model' state dict: %s" % path)
    scales = {}
    for name, qz in (blob.get("w_quantizers") or {}).items():
        s = _quantizer_scale(qz)
        if s is not None:
            scales[name] = s
    return blob["model"], scales


@torch.no_grad()
def int8_from_fake_quant(w: torch.Tensor, scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Real int8 codes ``[out, in]`` and fp32 scales ``[out]`` of a fake-quantised weight ``fp16(scale * code)``.

    With the quantiser's ``scale`` the codes are ``round(w / scale)`` (exact: the fp16 rounding of ``scale * code`` moves
    the quotient by less than 2**-11 * 128).  Without it the scale is recovered from the weight itself: a first guess
    absmax / 127 (the largest code of a row quantised without clipping is +-127), then one least-squares refit
    ``sum(w * c) / sum(c * c)``, which averages the fp16 rounding of the individual entries away.  Raises ``ValueError``
    when the result does not reproduce ``w`` to within one fp16 rounding: the weight was not int8 fake-quantised per row
    (or was clipped, in which case the quantiser's scale is required)."""
    wf = w.detach().float().flatten(1)
    if scale is None:
        s = wf.abs().amax(1).clamp(min=1e-5) / 127
        c = torch.round(wf / s[:, None]).clamp(-128, 127)
        den = (c * c).sum(1)
        s = torch.where(den > 0, (wf * c).sum(1) / den.clamp(min=1), s)
    else:
        s = scale.detach().float().flatten().to(wf.device)
        if s.numel() != wf.shape[0]:
            raise ValueError("one scale per output row expected: %d rows, %d scales" % (wf.shape[0], s.numel()))
    c = torch.round(wf / s[:, None]).clamp(-128, 127)
    back = (s[:, None] * c).to(w.dtype).float()
    ulp = wf.abs().clamp(min=2.0 ** -14) * 2.0 ** -10
    if not bool(((back - wf).abs() <= ulp).all()):
        raise ValueError("weight is not an int8 code times a per-row scale" + ("" if scale is not None else
                         " (clipped quantisation needs the quantiser's scale)"))
    return c.to(torch.int8).reshape(w.shape).contiguous(), s.contiguous()


_FFN_TARGETS = (("Ug", "gate_svd.BLinear"), ("Uu", "up_svd.BLinear"), ("Vg", "gate_svd.ALinear"), ("Vu", "up_svd.ALinear"),
                ("Wg", "gate_quant"), ("Wu", "up_quant"), ("Wd", "down_proj"))


def _find_weight(sd, prefix, target):
    """The weight of `target` and the quantiser key that goes with it: wrapped Linears appear as ``<t>.module.weight``."""
    for suffix in (".module", ""):
        key = "%s.%s%s.weight" % (prefix, target, suffix)
        if key in sd:
            return sd[key], "%s.%s%s" % (prefix, target, suffix)
    raise KeyError("no weight for %s.%s in the state dict" % (prefix, target))


def hybrid_ffn_weights(sd: Dict[str, torch.Tensor], prefix: str, scales: Optional[Dict[str, torch.Tensor]] = None,
                       online_had: Optional[bool] = None) -> dict:
    """The weight dict ``HybridFFN`` is built from, out of the entries ``<prefix>.*`` of a checkpoint's state dict
    (``prefix`` e.g. ``model.layers.3.mlp``; module layout of fake_quant/utils/hybrid_ffn_utils.py:923-954).  ``scales`` is
    the second result of ``load_qmodel``; its keys are looked up with and without a leading ``model.`` component since
    the reference names them ``model.layers.<i>.<target>`` whatever the state dict's own root is."""
    scales = scales or {}

    def scale_of(name):
        # the quantiser of a wrapped Linear is stored under the wrapper's name or under its `.module`, depending on the
        # target list (``mlp.gate_svd.BLinear`` but ``mlp.gate_quant.module``)
        for cand in (name, name[:-len(".module")] if name.endswith(".module") else name + ".module"):
            parts = cand.split(".")
            for start in range(len(parts)):
                if parts[start] == "layers":
                    k = "model." + ".".join(parts[start:])
                    if k in scales:
                        return scales[k]
            if cand in scales:
                return scales[cand]
        return None

    w = {}
    for short, target in _FFN_TARGETS:
        t, qname = _find_weight(sd, prefix, target)
        w[short + "_q"], w[short + "_s"] = int8_from_fake_quant(t, scale_of(qname))
    out = {"U_q": torch.cat([w["Ug_q"], w["Uu_q"]]), "U_s": torch.cat([w["Ug_s"], w["Uu_s"]])}
    for short in ("Vg", "Vu", "Wg", "Wu", "Wd"):
        out[short + "_q"], out[short + "_s"] = w[short + "_q"], w[short + "_s"]
    had_K = sd.get(prefix + ".had_K")
    K = 1
    if had_K is not None and had_K.dim() == 2:
        K = int(had_K.shape[0])
    else:
        had_K = None
    out["had_K"], out["K"] = had_K, K
    # the module sets ``online_had = had_K is not None`` when it is built (fake_quant/utils/hybrid_ffn_utils.py:947); the
    # attribute itself is not part of the state dict
    out["online_had"] = bool(online_had) if online_had is not None else had_K is not None
    perm = sd.get(prefix + ".perm")
    if perm is not None:
        out["perm"] = perm.to(torch.long)
    return out


def load_hybrid_ffn(path: str, prefix: str, device="cuda", online_had: Optional[bool] = None):
    """``HybridFFN`` for the FFN at ``prefix`` of a ``--save_qmodel_path`` checkpoint, on ``device``."""
    from .ffn import HybridFFN
    sd, scales = load_qmodel(path)
    w = hybrid_ffn_weights(sd, prefix, scales, online_had)
    w.pop("perm", None)
    return HybridFFN({k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in w.items()})
