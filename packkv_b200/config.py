"""Configuration carriers with the reference's names and semantics.

Mirrors utils/compute.py:6-20 (QuantMode, QuantMethod, RepackMethod) and
utils/config.py:22-141 (PackKVCacheConfig, ExtractCacheConfig) of the reference, so that
code written against the reference's cache configures this implementation unchanged.
"""
from __future__ import annotations

import ast
from enum import Enum


class QuantMode(Enum):
    BlockQuant = "BlockQuant"
    ChannelQuant = "ChannelQuant"
    TokenQuant = "TokenQuant"
    VectorQuant = "VectorQuant"


class QuantMethod(Enum):
    # (K mode, V mode)
    KIVI = (QuantMode.ChannelQuant, QuantMode.TokenQuant)
    PackKV = (QuantMode.TokenQuant, QuantMode.TokenQuant)


class RepackMethod(Enum):
    GREEDY = "Greedy"
    MEDIAN = "Median"
    NONE = "None"


class ExtractCacheConfig:
    """Collects raw K/V per generation round when quantisation is disabled."""

    def __init__(self, collect_round: int):
        self.collect_round = collect_round
        self.key_caches = {}
        self.value_caches = {}

    def size(self) -> int:
        total = 0
        for caches in (self.key_caches, self.value_caches):
            for per_round in caches.values():
                for t in per_round.values():
                    total += t.numel() * 16
        return total


class PackKVCacheConfig:
    _FIELDS = ("quant_method", "repack_method", "high_precision_zero_point", "block_size", "buffer_size",
               "pack_size", "k_quant_scale_rel", "v_quant_scale_rel")

    def __init__(self, model_name: str, quant_method, repack_method, high_precision_zero_point, block_size,
                 buffer_size, pack_size, k_quant_scale_rel, v_quant_scale_rel, enable_quant: bool = True):
        self.enable_quant = enable_quant
        self.model_name = model_name
        self.quant_method = quant_method
        self.repack_method = repack_method
        self.high_precision_zero_point = high_precision_zero_point
        self.block_size = block_size
        self.buffer_size = buffer_size
        self.pack_size = pack_size
        self.k_quant_scale_rel = k_quant_scale_rel
        self.v_quant_scale_rel = v_quant_scale_rel

    def _as_dict(self) -> dict:
        d = {"enable_quant": self.enable_quant, "model_name": self.model_name}
        if self.enable_quant:
            d["quant_method"] = self.quant_method.value
            d["repack_method"] = self.repack_method.value
            for f in self._FIELDS[2:]:
                d[f] = getattr(self, f)
        return d

    def __str__(self) -> str:
        return str(self._as_dict())

    __repr__ = __str__

    @staticmethod
    def from_str(text: str) -> "PackKVCacheConfig":
        """Inverse of str().  The reference evaluates the string as Python; here only
        literals and the enum constructors that str() emits are accepted."""
        import re

        def ev(node):
            if isinstance(node, ast.Dict):
                return {ev(k): ev(v) for k, v in zip(node.keys, node.values)}
            if isinstance(node, ast.Tuple):
                return tuple(ev(e) for e in node.elts)
            if isinstance(node, ast.Constant):
                return node.value
            raise ValueError("unsupported expression in config string")

        # enum members inside the quant_method tuple print as <QuantMode.X: 'X'>, which is not
        # Python; rewrite them to their string values before parsing
        cleaned = re.sub(r"<QuantMode\.\w+: '(\w+)'>", r"'\1'", text.strip())
        d = ev(ast.parse(cleaned, mode="eval").body)
        if d["enable_quant"]:
            qm = d["quant_method"]
            names = tuple(m if isinstance(m, str) else m.value for m in qm)
            quant_method = next(m for m in QuantMethod if tuple(x.value for x in m.value) == names)
            kwargs = dict(quant_method=quant_method, repack_method=RepackMethod(d["repack_method"]),
                          high_precision_zero_point=d["high_precision_zero_point"], block_size=d["block_size"],
                          buffer_size=d["buffer_size"], pack_size=d["pack_size"],
                          k_quant_scale_rel=d["k_quant_scale_rel"], v_quant_scale_rel=d["v_quant_scale_rel"])
        else:
            kwargs = dict(quant_method=None, repack_method=None, high_precision_zero_point=None, block_size=None,
                          buffer_size=None, pack_size=None, k_quant_scale_rel=None, v_quant_scale_rel=None)
        return PackKVCacheConfig(model_name=d["model_name"], enable_quant=d["enable_quant"], **kwargs)

    def _key(self):
        return (self.enable_quant, self.model_name, self.quant_method, self.repack_method,
                self.high_precision_zero_point, self.block_size, self.buffer_size, self.pack_size,
                self.k_quant_scale_rel, self.v_quant_scale_rel)

    def __eq__(self, other) -> bool:
        return isinstance(other, PackKVCacheConfig) and self._key() == other._key()

    def __hash__(self) -> int:
        return hash(self._key())
