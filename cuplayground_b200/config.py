"""Layer configuration: the keys of the reference's aristos_config.json (aristos_config.json:1-13, validated by
aristos_config.schema.json:1-71) plus the extension keys of include/aristos_moe.h. Parsing and validation happen in
the C library; this class only carries the values across the ABI."""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import asdict, dataclass

from . import _lib


@dataclass
class AristosConfig:
    # reference keys (defaults = the shipped aristos_config.json)
    capacity_factor: float = 1.0
    drop_tokens: int = 0
    expert_top_k: int = 1
    is_training: int = 0
    hidden_act: int = 0
    hidden_size: int = 1024
    intermediate_size: int = 4096
    micro_batch: int = 4
    num_experts: int = 1
    sequence_len: int = 2048
    torch_dtype: int = 0
    # extension keys
    tokens: int = 0
    gate_fn: int = 0
    renorm_topk: int = 0
    gate_bias_zipf_s: float = 0.0
    ep_world: int = 1
    seed: int = 0

    def to_struct(self) -> _lib.AristosConfigStruct:
        s = _lib.AristosConfigStruct()
        for k, v in asdict(self).items():
            setattr(s, k, v)
        return s

    @classmethod
    def from_struct(cls, s: _lib.AristosConfigStruct) -> "AristosConfig":
        return cls(**{name: getattr(s, name) for name, _ in s._fields_})

    @classmethod
    def from_json(cls, text: str) -> "AristosConfig":
        s = _lib.AristosConfigStruct()
        _lib.check(_lib.load().aristos_config_parse(text.encode(), C.byref(s)))
        return cls.from_struct(s)

    @classmethod
    def load(cls, path: str) -> "AristosConfig":
        s = _lib.AristosConfigStruct()
        _lib.check(_lib.load().aristos_config_load(str(path).encode(), C.byref(s)))
        return cls.from_struct(s)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2)

    def validate(self) -> None:
        s = self.to_struct()
        _lib.check(_lib.load().aristos_config_validate(C.byref(s)))

    @property
    def S(self) -> int:
        s = self.to_struct()
        return int(_lib.load().aristos_config_tokens(C.byref(s)))

    @property
    def capacity(self) -> int:
        s = self.to_struct()
        return int(_lib.load().aristos_config_capacity(C.byref(s)))


def baseline_config(n: int, world: int = 1) -> AristosConfig:
    """The five benchmark configurations (1-based): fp32 reference case, single-GPU GELU, Mixtral-shaped SwiGLU,
    DeepSeek-V3-shaped FP8, skewed routing."""
    if n == 1:
        return AristosConfig(capacity_factor=1.0, drop_tokens=1, expert_top_k=1, hidden_act=0, hidden_size=256,
                             intermediate_size=512, num_experts=8, torch_dtype=0, tokens=128, seed=0, ep_world=world)
    if n == 2:
        return AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=1, hidden_size=2048,
                             intermediate_size=2048, num_experts=64, torch_dtype=2, tokens=8192, renorm_topk=1,
                             seed=1, ep_world=world)
    if n == 3:
        return AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=2, hidden_size=4096,
                             intermediate_size=14336, num_experts=8, torch_dtype=2, tokens=16384, seed=2,
                             ep_world=world)
    if n == 4:
        return AristosConfig(capacity_factor=1.0, drop_tokens=0, expert_top_k=8, hidden_act=2, hidden_size=7168,
                             intermediate_size=2048, num_experts=256, torch_dtype=4, tokens=4096, gate_fn=1,
                             renorm_topk=1, seed=3, ep_world=world)
    if n == 5:
        return AristosConfig(capacity_factor=1.0, drop_tokens=1, expert_top_k=4, hidden_act=1, hidden_size=2048,
                             intermediate_size=1024, num_experts=128, torch_dtype=2, tokens=8192,
                             gate_bias_zipf_s=1.2, seed=4, ep_world=world)
    raise ValueError("configurations are numbered 1..5")
