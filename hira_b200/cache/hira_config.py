"""HiraConfig / DeviceMode with the reference's fields and kwargs getters
(cache/hira_config.py:5-46).  `from_dict` / `from_yaml`, which the reference leaves
unimplemented (:27-33), are provided; the extra fields configure this build only."""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional


@dataclass
class DeviceMode:
    CPU_ONLY = "cpu_only"
    CUDA_ONLY = "cuda_only"
    CPU_CUDA = "cpu-cuda"


@dataclass
class HiraConfig:
    # cache
    device_mode: str = DeviceMode.CPU_ONLY  # reference default; this build runs "cuda_only"
    update_every: int = 1
    # indexers
    num_levels: int = 5  # reference default; the CUDA index supports 2 or 3
    max_iterations: int = 1
    branching_factor: int = 10
    # threshold
    threshold_method: str = "sample_mean_topk"  # "sample_max" or "sample_mean_topk"
    sample_size: int = 1000
    topk: int = 16
    # searcher
    chunk_size = 8 * 1024
    # this build
    max_context: Optional[int] = None  # pre-allocate the index for this many keys per head
    gate: str = "ge"                   # tree gate used by hira_attention: "ge" or "gt"
    use_tensor_cores: bool = True
    balance_rounds: int = 0            # capacity-aware assignment rounds of the index build (0: the reference's rule)

    @classmethod
    def from_dict(cls, config_dict: dict) -> "HiraConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(config_dict) - known - {"chunk_size"}
        if unknown:
            raise ValueError(f"unknown HiraConfig keys: {sorted(unknown)}")
        cfg = cls(**{k: v for k, v in config_dict.items() if k in known})
        if "chunk_size" in config_dict:
            cfg.chunk_size = config_dict["chunk_size"]
        return cfg

    @classmethod
    def from_yaml(cls, config_path: str) -> "HiraConfig":
        import yaml
        with open(config_path) as f:
            data = yaml.safe_load(f) or {}
        if "hira" in data and isinstance(data["hira"], dict):
            data = data["hira"]
        return cls.from_dict(data)

    def get_indexer_kwargs(self) -> dict:
        kw = {
            "num_levels": self.num_levels,
            "max_iterations": self.max_iterations,
            "branching_factor": self.branching_factor,
        }
        if self.device_mode == DeviceMode.CUDA_ONLY:
            if self.max_context is not None:
                kw["max_context"] = self.max_context
            if not self.use_tensor_cores:
                kw["use_tensor_cores"] = False
            if self.balance_rounds:
                kw["balance_rounds"] = self.balance_rounds
        return kw

    def get_searcher_kwargs(self) -> dict:
        if self.device_mode == DeviceMode.CUDA_ONLY:
            return {"block_c": self.branching_factor}
        return {"chunk_size": self.chunk_size}
