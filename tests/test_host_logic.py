"""CPU-only checks: the C ABI library loads and exports every declared symbol, the config and
cache host logic behaves like the reference's (tests/test_hira_cache.py there), and the
multi-rank plumbing works over gloo."""
import ctypes
import os
import re
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    from hira_b200 import _lib
    lib = _lib.load()
    header = (ROOT / "include" / "hira_b200.h").read_text()
    declared = set(re.findall(r"\b(hira_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/hira_b200.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= declared
    assert b"sm_100a" in lib.hira_version()


def test_argument_errors_are_reported_without_a_gpu():
    from hira_b200 import _lib
    lib = _lib.load()
    ix = _lib.HiraIndexStruct()          # all zero: invalid depth, bf, dim ...
    rc = lib.hira_search(ctypes.byref(ix), None, None, None, None, None, 1, 0, 0, 1, None, None, None, None, None, None)
    assert rc < 0 and lib.hira_last_error()
    with pytest.raises(ValueError):
        _lib.check(rc, "hira_search")
    assert lib.hira_build_workspace_bytes(ctypes.byref(ix), 10) == 0
    assert lib.hira_attn_default_splits(512, 128) >= 1
    # the peer exchange: buffer size = 2 parities x world x heads x ((2 + V) floats + one flag); host-side refusals
    assert lib.hira_exchange_bytes(8, 64, 128) == 2 * 8 * 64 * ((128 + 2) * 4 + 4)
    assert lib.hira_exchange_bytes(0, 64, 128) == 0
    rc = lib.hira_exchange_merge(None, None, 2, 0, 8, 64, 1, 3, 0.0, None, None, None, None)
    assert rc == _lib.HIRA_ERR_ARG and b"NULL" in lib.hira_last_error()
    assert lib.hira_q8_fallback_count(None) == _lib.HIRA_ERR_ARG


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from hira_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_config_defaults_and_kwargs_match_reference():
    from hira_b200 import DeviceMode, HiraConfig
    c = HiraConfig()
    # cache/hira_config.py:12-24
    assert (c.device_mode, c.update_every, c.num_levels, c.max_iterations, c.branching_factor) == ("cpu_only", 1, 5, 1, 10)
    assert (c.threshold_method, c.sample_size, c.chunk_size) == ("sample_mean_topk", 1000, 8 * 1024)
    assert c.get_indexer_kwargs() == {"num_levels": 5, "max_iterations": 1, "branching_factor": 10}
    assert c.get_searcher_kwargs() == {"chunk_size": 8 * 1024}
    g = HiraConfig(device_mode=DeviceMode.CUDA_ONLY, num_levels=3, branching_factor=32, max_context=1000)
    assert g.get_searcher_kwargs() == {"block_c": 32}
    assert g.get_indexer_kwargs()["max_context"] == 1000


def test_config_from_dict_and_yaml(tmp_path):
    from hira_b200 import HiraConfig
    c = HiraConfig.from_dict({"device_mode": "cuda_only", "num_levels": 2, "branching_factor": 16, "chunk_size": 64})
    assert (c.device_mode, c.num_levels, c.branching_factor, c.chunk_size) == ("cuda_only", 2, 16, 64)
    with pytest.raises(ValueError):
        HiraConfig.from_dict({"no_such_field": 1})
    p = tmp_path / "c.yml"
    p.write_text("hira:\n  device_mode: cuda_only\n  update_every: 4\n  num_levels: 3\n")
    y = HiraConfig.from_yaml(str(p))
    assert (y.device_mode, y.update_every, y.num_levels) == ("cuda_only", 4, 3)


class _DummyIndexer:
    def __init__(self, **kw):
        self.kw, self.built, self.updates = kw, None, []

    def build(self, k, v):
        self.built = (k, v)
        return self

    def update(self, k, v):
        self.updates.append((k.clone(), v.clone()))
        return self


class _DummySearcher:
    def __init__(self, **kw):
        self.kw = kw


class _Cfg:
    num_hidden_layers = 3

    def get_text_config(self, decoder=True):
        return self


def _layer(monkeypatch, update_every):
    import hira_b200.cache.hira_cache as hc
    monkeypatch.setattr(hc, "CUDAIndexer", _DummyIndexer)
    monkeypatch.setattr(hc, "CUDASearcher", _DummySearcher)
    from hira_b200 import HiraConfig
    cfg = HiraConfig(device_mode="cuda_only", update_every=update_every, num_levels=3, branching_factor=8)
    return hc, cfg


def test_cache_prefill_queue_and_flush(monkeypatch):
    hc, cfg = _layer(monkeypatch, update_every=3)
    cache = hc.HiraCache(_Cfg(), cfg)
    assert len(cache.layers) == 3
    k, v = torch.randn(1, 2, 10, 16), torch.randn(1, 2, 10, 16)
    out, none = cache.update(k, v, 1)
    assert none is None and isinstance(out, hc.CacheOutput)
    assert out.prefill_keys is k and out.prefill_values is v
    assert tuple(out.queued_keys.shape) == (1, 2, 0, 16)
    assert out.indexer.kw == {"num_levels": 3, "max_iterations": 1, "branching_factor": 8}
    assert out.searcher.kw == {"block_c": 8}
    assert cache.get_seq_length(1) == 10 and cache.get_seq_length(0) == 0
    for i in range(2):
        out, _ = cache.update(torch.full((1, 2, 1, 16), float(i)), torch.full((1, 2, 1, 16), float(i)), 1)
        assert out.prefill_keys is None and out.queued_keys.shape[2] == i + 1 and not out.indexer.updates
    out, _ = cache.update(torch.full((1, 2, 1, 16), 2.0), torch.full((1, 2, 1, 16), 2.0), 1)
    assert out.queued_keys.shape[2] == 0 and len(out.indexer.updates) == 1
    assert out.indexer.updates[0][0][0, 0, :, 0].tolist() == [0.0, 1.0, 2.0]       # the whole queue, in order
    assert cache.get_seq_length(1) == 13
    assert cache.layers[1].get_mask_sizes(1) == (14, 0)
    assert cache.layers[1].get_mask_sizes(torch.arange(2)) == (15, 0)
    cache.layers[1].reset()
    assert cache.get_seq_length(1) == 0


def test_cpu_device_mode_is_refused():
    from hira_b200 import HiraCacheLayer
    with pytest.raises(NotImplementedError):
        HiraCacheLayer("cpu_only", 1, {}, {})


def test_layer_count_follows_the_model_config(monkeypatch):
    hc, cfg = _layer(monkeypatch, 1)

    class Sliding(_Cfg):
        sliding_window = 128
        num_hidden_layers = 5
        num_kv_shared_layers = 2
    assert len(hc.HiraCache(Sliding(), cfg).layers) == 3


def test_head_and_sequence_sharding():
    from hira_b200.parallel import shard_heads, shard_sequence
    for world in (1, 2, 4, 8):
        owned = [list(shard_heads(8, world, r)) for r in range(world)]
        assert sorted(sum(owned, [])) == list(range(8)) and all(len(o) == 8 // world for o in owned)
    assert [len(shard_heads(10, 4, r)) for r in range(4)] == [3, 3, 2, 2]
    spans = [shard_sequence(1_048_576, 8, r) for r in range(8)]
    assert spans[0] == (0, 131072) and spans[-1] == (917504, 1048576)
    with pytest.raises(ValueError):
        shard_heads(8, 2, 2)


def _gloo_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from hira_b200.parallel import gather_partials, shard_sequence
    from oracle import oracle as O
    g = torch.Generator().manual_seed(0)
    hq, n, d = 4, 64, 16
    logits = torch.randn((hq, n), generator=g) * 3
    vals = torch.randn((n, d), generator=g)
    lo, hi = shard_sequence(n, world, rank)
    m = logits[:, lo:hi].max(dim=1).values
    p = torch.exp(logits[:, lo:hi] - m[:, None])
    l = p.sum(dim=1)
    o = (p @ vals[lo:hi]) / l[:, None]
    po, pml = gather_partials(o.contiguous(), torch.stack([m, l], dim=1).contiguous())
    merged, _ = O.merge_partials(po.numpy(), pml.numpy())
    full = torch.softmax(logits, dim=1) @ vals
    err = float(np.abs(merged - full.numpy()).max())
    # the same through the preallocated exchange buffer: the partials are written in place
    # (strided views of this rank's slice), gathered in place, and read back through strides
    from hira_b200.parallel import PartialsExchange
    ex = PartialsExchange(hq, d, "cpu")
    assert ex.world == world and ex.message_bytes == hq * (d + 2) * 4
    ex.local_out.copy_(o)
    ex.local_ml.copy_(torch.stack([m, l], dim=1))
    buf = ex.all_gather()
    merged2, _ = O.merge_partials(np.ascontiguousarray(buf[:, :, 2:].numpy()), np.ascontiguousarray(buf[:, :, :2].numpy()))
    ret[rank] = max(err, float(np.abs(merged2 - full.numpy()).max()))
    dist.destroy_process_group()


def test_sequence_shard_partials_gather_over_gloo():
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_gloo_worker, args=(2, port, ret), nprocs=2, join=True)
        assert len(ret) == 2 and max(ret.values()) < 1e-5
