"""Host logic of the autotuner (candidate lists, table keys, persistence, locking) without a GPU."""

import json
import threading

import torch

from mxblas_b200 import MxbConfig, tune
from mxblas_b200.mx_gemm import get_meta_info


def _meta(m, n, k, sm, sn, sk, quant=False, qn=16):
    e4, f32 = torch.float8_e4m3fn, torch.float32
    return get_meta_info(e4, e4, f32, f32, quant, (1, qn) if quant else None, None, (m, k), (k, n), (m // sm, k // sk),
                         (k // sk, n // sn), (k, 1), (1, k), (k // sk, 1), (1, k // sk), False, False)


def test_candidates_cover_the_kernel_families():
    """Every family the heuristic plan can pick is among the candidates: CTA pairs for all three scale modes,
    the K-sliced last wave on and off, and the heuristic plan itself as the first candidate."""
    big = tune.candidates(8192, 8192, 8192, 8192, True, False, False)
    assert big[0].key() == tune.AUTO
    assert any(c.cta_pair == 2 for c in big) and any(c.cta_pair == 1 and c.bn == 256 for c in big)
    assert {c.splits for c in big if c.cta_pair == 2} >= {0, 1}
    skinny = tune.candidates(16, 28672, 8192, 8192, False, False, False)
    assert all(c.swap == 1 for c in skinny[1:]) and {c.splits for c in skinny} >= {1, 2, 3}
    assert any(c.bn == 32 for c in skinny)
    promote = tune.candidates(4096, 7168, 7168, 128, False, False, False)
    assert {(c.bn, c.epi_warps, c.cta_pair) for c in promote} >= {(128, 8, 1), (256, 8, 1), (256, 8, 2)}
    mx = tune.candidates(16384, 1024, 8192, 32, True, True, True)
    assert all(c.swap == 1 for c in mx[1:]) and {c.bn for c in mx[1:]} == {128, 224}
    assert any(c.cta_pair == 2 and c.bn == 224 for c in mx)


def test_table_key_buckets_m_and_roundtrips(tmp_path, monkeypatch):
    monkeypatch.setenv("MXBLAS_CACHE_DIR", str(tmp_path))
    tune.reload_tables()
    a, b = _meta(48, 4096, 4096, 1, 1, 4096), _meta(64, 4096, 4096, 1, 1, 4096)
    assert tune.table_key(a, False, None) == tune.table_key(b, False, None)  # same M bucket
    assert tune.table_key(a, False, None) != tune.table_key(_meta(128, 4096, 4096, 1, 1, 4096), False, None)
    assert tune.table_key(a, False, None) != tune.table_key(a, True, None)
    assert tune.lookup(a, False, None) is None
    tune._load_table()[tune.table_key(a, False, None)] = {"config": [64, 1, 4, 8, 2, 0, 1], "us": 12.5}
    tune._save_table()
    tune.reload_tables()  # a new process would start like this: nothing in memory, the file on disk
    got = tune.lookup(b, False, None)
    assert isinstance(got, MxbConfig) and got.key() == (64, 1, 4, 8, 2, 0, 1)
    assert tune.plan_for(b, False, None).key() == got.key()
    assert json.loads(tune._table_path().read_text())
    tune.reload_tables()


def test_heuristic_winner_is_stored_but_not_forced(tmp_path, monkeypatch):
    """When the heuristic plan wins, the table remembers that the problem was tuned, and calls keep passing no
    configuration (so later improvements of the heuristic are not frozen out)."""
    monkeypatch.setenv("MXBLAS_CACHE_DIR", str(tmp_path))
    tune.reload_tables()
    a = _meta(512, 4096, 4096, 1, 1, 4096)
    tune._load_table()[tune.table_key(a, False, None)] = {"config": list(tune.AUTO), "us": 30.0}
    assert tune.lookup(a, False, None) is None and tune.table_key(a, False, None) in tune._load_table()
    tune.reload_tables()


def test_concurrent_saves_keep_every_entry(tmp_path, monkeypatch):
    """Threads that store winners at the same time (the table's lock) and a second writer's file on disk
    (merged on save) all survive."""
    monkeypatch.setenv("MXBLAS_CACHE_DIR", str(tmp_path))
    tune.reload_tables()
    path = tune._table_path()
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps({"other-process": {"config": [128, 0, 4, 8, 1, 0, 1], "us": 1.0}}))
    tune.reload_tables()

    def store(i):
        with tune._lock:
            tune._load_table()[f"k{i}"] = {"config": [256, 0, 4, 8, 1, 0, 2], "us": float(i)}
            tune._save_table()

    threads = [threading.Thread(target=store, args=(i,)) for i in range(16)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    on_disk = json.loads(path.read_text())
    assert set(on_disk) == {"other-process"} | {f"k{i}" for i in range(16)}
    tune.reload_tables()


def test_m_bucket():
    assert [tune.m_bucket(m) for m in (1, 16, 17, 64, 65, 4096)] == [16, 16, 32, 64, 128, 4096]
