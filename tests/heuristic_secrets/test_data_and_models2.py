"""Data builder, collectors, synthetic tasks, ByteMasker and Joint detector (CPU)."""
import torch

from ml_experiments_b200.heuristic_secrets.bytemasker.model import ByteMaskerConfig, ByteMaskerModel
from ml_experiments_b200.heuristic_secrets.data import synthetic as S
from ml_experiments_b200.heuristic_secrets.data.build import DataBuilder
from ml_experiments_b200.heuristic_secrets.data.collectors.generated import Base64Generator, HashGenerator, UUIDGenerator
from ml_experiments_b200.heuristic_secrets.data.collectors.scrapers import FixtureScraper, extract_literals, infer_category
from ml_experiments_b200.heuristic_secrets.data.pipeline import deduplicate_samples, read_jsonl, split_samples
from ml_experiments_b200.heuristic_secrets.data.registry import CollectorRegistry, get_default_registry
from ml_experiments_b200.heuristic_secrets.data.types import CATEGORY_LABELS, SecretCategory, SpanFinderSample, ValidatorSample
from ml_experiments_b200.heuristic_secrets.joint import JointConfig, JointSecretDetector
from ml_experiments_b200.heuristic_secrets.validator import FrequencyTable


def test_generators_and_registry():
    u = list(UUIDGenerator(count=10, seed=0).collect())
    assert len(u) == 10 and all(len(s.text) == 36 and s.label == 0 and s.category == "fp_uuid" for s in u)
    assert [s.text for s in UUIDGenerator(count=10, seed=0).collect()] == [s.text for s in u]
    assert all(len(s.text) == n for ht, n in (("md5", 32), ("sha1", 40), ("sha256", 64)) for s in HashGenerator(ht, 5, seed=1).collect())
    assert all(20 <= len(s.text) <= 104 for s in Base64Generator(count=20, seed=2).collect())
    names = get_default_registry().names()
    assert {"generated_uuids", "generated_md5", "generated_sha1", "generated_sha256", "generated_base64", "detect_secrets",
            "gitleaks", "trufflehog", "creddata"} <= set(names)
    assert len(SecretCategory) == 12 and CATEGORY_LABELS[SecretCategory.API_KEY] == 1 and CATEGORY_LABELS[SecretCategory.FP_HASH] == 0


def test_scraper_and_builder(tmp_path):
    (tmp_path / "repo" / "tests").mkdir(parents=True)
    (tmp_path / "repo" / "tests" / "fixtures.go").write_text(
        'apiKey := "AKIAIOSFODNN7EXAMPLE12"\nvar password = "Tr0ub4dor&3xyz"\nmsg := "plain english sentence here ok"\n')
    lits = extract_literals('token = "ghp_abcDEF1234567890xyz"')
    assert lits[0][2] == "ghp_abcDEF1234567890xyz" and infer_category("token", lits[0][2]) == SecretCategory.AUTH_TOKEN

    class Local(FixtureScraper):
        name = "local"

    reg = CollectorRegistry()
    reg.register(Local, root=tmp_path / "repo")
    reg.register(UUIDGenerator, count=40, seed=0)
    res = DataBuilder(tmp_path / "out", registry=reg, seed=1, no_fetch=True).build()
    assert {k: v["samples"] for k, v in res.sources.items()} == {"local": 2, "generated_uuids": 40} and res.sources["local"]["spans"] == 1
    assert sum(res.splits["validator"].values()) == 42 and res.deduplication == {"validator_before": 42, "validator_after": 42}
    train = list(read_jsonl(tmp_path / "out" / "splits" / "validator" / "train.jsonl", ValidatorSample))
    assert len(train) == res.splits["validator"]["train"]
    import json
    on_disk = json.loads((tmp_path / "out" / "manifest.json").read_text())
    assert {"created_at", "sources", "splits", "deduplication"} <= set(on_disk) and on_disk["splits"] == res.splits
    assert DataBuilder(tmp_path / "o2", sources=["generated_uuids", "no_such_source"], no_fetch=True).registry.names() == ["generated_uuids"]
    docs = [s for split in ("train", "val", "test") for s in read_jsonl(tmp_path / "out" / "splits" / "documents" / f"{split}.jsonl", SpanFinderSample)]
    assert len(docs) == 1 and len(docs[0].starts) == 2
    raw = docs[0].text.encode()
    assert raw[docs[0].starts[0]:docs[0].ends[0]] == b"AKIAIOSFODNN7EXAMPLE12"


def test_split_and_dedupe():
    samples = [ValidatorSample(f"s{i % 50}", i % 2, "x", "api_key" if i % 2 else "fp_uuid") for i in range(120)]
    d = deduplicate_samples(samples)
    assert len(d) == 50
    tr, va, te = split_samples(d, seed=0)
    assert len(tr) + len(va) + len(te) == 50 and {s.category for s in tr} == {"api_key", "fp_uuid"}
    assert [s.text for s in split_samples(d, seed=0)[0]] == [s.text for s in tr]


def test_synthetic_tasks():
    for name, fn in S.TASKS.items():
        d = fn(seq_len=32, num_examples=50, seed=0)
        assert d.inputs.shape == (50, 32) == d.labels.shape and d.task == name
    m = S.mqar(vocab_size=64, seq_len=32, num_kv_pairs=4, num_examples=20, seed=1)
    for x, y in zip(m.inputs, m.labels):
        kv = dict(zip(x[0:8:2].tolist(), x[1:8:2].tolist()))
        assert (y[:-4] == -100).all() and all(kv[q] == a for q, a in zip(x[-4:].tolist(), y[-4:].tolist()))
    p = S.cumulative_parity(seq_len=16, num_examples=5, seed=2)
    assert torch.equal(p.labels, p.inputs.cumsum(1) % 2)
    c = S.selective_copying(vocab_size=32, seq_len=40, num_tokens=6, num_examples=10, seed=3)
    for x, y in zip(c.inputs, c.labels):
        assert x[x < 30][:6].tolist() == y[-6:].tolist()
    tr, te, cfg = S.load_task("induction_heads", seq_len=24, num_train=64, num_test=32, batch_size=16)
    xb, yb = next(iter(tr))
    assert xb.shape == (16, 24) and cfg["vocab_size"] == 256


def test_bytemasker_and_joint():
    torch.manual_seed(0)
    m = ByteMaskerModel(ByteMaskerConfig.tiny())
    x = torch.randint(0, 256, (3, 60))
    logits, h = m(x, return_hidden=True)
    assert logits.shape == (3, 60) and h.shape == (3, 60, 32) and m.predict(x).shape == (3, 60)
    assert ByteMaskerConfig.from_dict(ByteMaskerConfig.medium().to_dict()) == ByteMaskerConfig.medium()
    j = JointSecretDetector(JointConfig.default(), FrequencyTable.from_data(b"plain text"), FrequencyTable.from_data(b"A1b2C3d4"))
    out = j(x, torch.tensor([60, 10, 3]))
    assert out["cls_logits"].shape == (3, 1) and (out["pruned_lengths"] >= 3).all() and out["pruned_lengths"][2] == 3
    (out["cls_logits"].sum() + out["mask_logits"].sum()).backward()
    assert JointConfig.from_dict(JointConfig.default().to_dict()).to_dict() == JointConfig.default().to_dict()
