"""Checkpoint container and catalog: strict validation, sparse-file offsets beyond 4 GiB, official-layout round trip."""
import json
import os
import struct

import pytest
import torch

from ds41rt_b200.config import ModelConfig
from ds41rt_b200.loader import Catalog, SafetensorsError, SafetensorsFile, expected_tensors, official_templates, \
    write_safetensors
from ds41rt_b200.loader.official import export_official, load_official
from ds41rt_b200.models.weights import init_weights


def _raw(path, header: dict, data_len: int):
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        f.truncate(8 + len(h) + data_len)


def test_roundtrip_and_slices(tmp_path):
    p = str(tmp_path / "a.safetensors")
    a = torch.arange(6 * 8, dtype=torch.float32).view(6, 8)
    b = torch.randn(5, 4).bfloat16()
    write_safetensors(p, {"a": a, "b": b, "s": torch.tensor(3.5)})
    f = SafetensorsFile(p)
    assert torch.equal(f.read("a"), a) and torch.equal(f.read("b"), b) and float(f.read("s")) == 3.5
    assert torch.equal(f.read("a", rows=(2, 5)), a[2:5])
    assert torch.equal(f.read("a", cols=(3, 7)), a[:, 3:7])
    assert torch.equal(f.read("a", rows=(1, 4), cols=(2, 6)), a[1:4, 2:6])
    with pytest.raises(SafetensorsError):
        f.read("a", rows=(0, 7))


def test_adversarial_headers(tmp_path):
    p = str(tmp_path / "x.safetensors")
    ok = {"t": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}
    _raw(p, ok, 16)
    SafetensorsFile(p)
    _raw(p, ok, 20)                                             # trailing bytes
    with pytest.raises(SafetensorsError, match="trailing"):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, 12)          # length mismatch
    with pytest.raises(SafetensorsError, match="does not match"):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
             "u": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, 6)               # overlap
    with pytest.raises(SafetensorsError, match="gap or overlaps"):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, 8)               # gap at start
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 4]}}, 4)
    with pytest.raises(SafetensorsError, match="unknown dtype"):
        SafetensorsFile(p)
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="implausible"):
        SafetensorsFile(p)


def test_sparse_file_offsets_beyond_4gib(tmp_path):
    p = str(tmp_path / "big.safetensors")
    big = 5 * (1 << 30)
    hdr = {"pad": {"dtype": "U8", "shape": [big], "data_offsets": [0, big]},
           "tail": {"dtype": "F32", "shape": [4, 4], "data_offsets": [big, big + 64]}}
    _raw(p, hdr, big + 64)
    want = torch.arange(16, dtype=torch.float32).view(4, 4)
    f = SafetensorsFile(p)
    with open(p, "r+b") as fh:
        fh.seek(f.data_start + big)
        fh.write(want.numpy().tobytes())
    assert torch.equal(f.read("tail"), want)
    assert torch.equal(f.read("tail", rows=(1, 3), cols=(1, 4)), want[1:3, 1:4])


def test_official_flash_catalog_shape():
    cfg = ModelConfig.flash()
    want = expected_tensors(cfg)
    assert want["layers.0.attn.wq_b.weight"] == ("F8_E4M3", (32768, 1280))
    assert want["layers.0.attn.wo_a.scale"] == ("F8_E8M0", (256, 128))
    assert want["layers.5.ffn.experts.383.w2.weight"] == ("I8", (5120, 1152))
    assert want["layers.1.engram.wkv.weight"] == ("F8_E4M3", (25600, 6144))
    assert want["mtp.0.main_proj.scale"] == ("F8_E8M0", (160, 480))
    assert want["aligner.w1.weight"] == ("BF16", (5120, 9216))
    assert len(want) == 96085                       # tensor count of the official checkpoint
    assert len(official_templates(cfg)) == 116


def test_official_layout_roundtrip_and_strict_catalog(tmp_path):
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=0)
    d = str(tmp_path / "ckpt")
    export_official(cfg, w, d, shards=3)
    cat = Catalog(d, cfg, with_vision=False, with_engram=False)
    got = load_official(cat)
    for name in ("layers.0.attn.wq_a.weight", "layers.1.ffn.experts.3.w1.weight", "embed.weight", "layers.0.hc_attn_fn"):
        ref = w[name]
        err = float((got[name] - ref).abs().max())
        tol = 0.26 * float(ref.abs().max()) if ".experts." in name else 0.07 * float(ref.abs().max()) + 1e-3
        assert err <= tol, (name, err)
    # one rank's shard of two: sliced shapes and only its experts
    part = load_official(cat, rank=1, world=2)
    assert part["layers.0.attn.wq_b.weight"].shape == (cfg.n_heads // 2 * cfg.head_dim, cfg.q_lora)
    assert torch.equal(part["layers.0.attn.wq_b.weight"], got["layers.0.attn.wq_b.weight"][512:])
    assert part["layers.0.attn.wo_b.weight"].shape == (cfg.hidden, cfg.o_lora)
    assert "layers.0.ffn.experts.3.w1.weight" not in part and "layers.0.ffn.experts.12.w1.weight" in part
    assert cat.shard_bytes(0, 2) < sum(e.nbytes for f in cat.files.values() for e in f.entries.values())
    # strictness: a renamed tensor is both "missing" and "unknown"
    idx = os.path.join(d, "model.safetensors.index.json")
    doc = json.load(open(idx))
    doc["weight_map"]["bogus.weight"] = doc["weight_map"].pop("norm.weight")
    json.dump(doc, open(idx, "w"))
    with pytest.raises(SafetensorsError):
        Catalog(d, cfg, with_vision=False, with_engram=False)


def test_nvfp4_variant_catalog(tmp_path):
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=1)
    d = str(tmp_path / "nv")
    export_official(cfg, w, d, variant="nvfp4", shards=1)
    cat = Catalog(d, cfg, variant="nvfp4", with_vision=False, with_engram=False)
    got = load_official(cat)
    ref = w["layers.0.ffn.experts.0.w2.weight"]
    assert float((got["layers.0.ffn.experts.0.w2.weight"] - ref).abs().max()) < 0.2 * float(ref.abs().max())
    with pytest.raises(SafetensorsError):
        Catalog(d, cfg, variant="mxfp4", with_vision=False, with_engram=False)


def test_lazy_weights_match_eager_load(tmp_path):
    """The streaming view used to fill engine shards returns exactly what the eager loader returns."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.loader.official import LazyOfficialWeights
    from ds41rt_b200.models.weights import init_weights
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=3)
    d = str(tmp_path / "ckpt")
    export_official(cfg, w, d, shards=2)
    cat = Catalog(d, cfg, with_vision=False, with_engram=False)
    eager = load_official(cat)
    lazy = LazyOfficialWeights(cat)
    for name in ("embed.weight", "layers.0.attn.wq_a.weight", "layers.1.ffn.experts.3.w1.weight", "layers.0.hc_attn_fn"):
        assert name in lazy
        assert torch.equal(lazy[name], eager[name])


def test_engram_table_export_matches_checkpoint_rows(tmp_path):
    """An Engram layer of an official-layout checkpoint: the exported flat table holds the checkpoint's e4m3 payload and
    UE8M0 scales record by record, and dequantises to the stored values."""
    import dataclasses
    import numpy as np
    from ds41rt_b200.config import EngramConfig
    from ds41rt_b200.loader.official import export_engram_table
    from ds41rt_b200.models.engram import dequant_rows_reference
    from ds41rt_b200.runtime.engram_io import EngramTable
    cfg = dataclasses.replace(ModelConfig.tiny(), engram=EngramConfig(layers=(1,), num_embeddings=(3000,)))
    w = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    H, width = cfg.hidden, 24 * 256
    w["layers.1.engram.embed.weight"] = torch.randn(3000, 256, generator=g)
    w["layers.1.engram.k_weight"] = torch.randn(cfg.hc_mult, H, generator=g)
    w["layers.1.engram.q_weight"] = torch.randn(cfg.hc_mult, H, generator=g)
    w["layers.1.engram.wkv.weight"] = torch.randn((cfg.hc_mult + 1) * H, width, generator=g) * 0.02
    d = str(tmp_path / "ckpt")
    export_official(cfg, w, d, shards=2, with_engram=True)
    cat = Catalog(d, cfg, with_vision=False, with_engram=True)
    path = str(tmp_path / "engram1.bin")
    assert export_engram_table(cat, 1, path, chunk_rows=1024) == 3000
    table = EngramTable(path, 3000, 264)
    rec = torch.from_numpy(np.fromfile(path, dtype=np.uint8).reshape(3000, 264))
    deq = dequant_rows_reference(rec, 256)
    ref = w["layers.1.engram.embed.weight"]
    assert float((deq - ref).abs().max()) <= 0.07 * float(ref.abs().max())
    table.close()


def test_fp4_experts_import_byte_for_byte(tmp_path):
    """An FP4 + UE8M0/32 checkpoint becomes the engine's MX-FP4 expert stacks without dequantising a value: payload
    bytes are the checkpoint's, the scales are only re-tiled into 128 x 4 atoms; the stacks expand to exactly the
    values the dequantising loader reads."""
    from ds41rt_b200.loader.official import LazyOfficialWeights
    from ds41rt_b200.models.ds41 import EngineWeights, dequantize_expert_fp4
    from ds41rt_b200.ops.mx import pack_sf_atoms, pack_sf_atoms_batched
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=3)
    d = str(tmp_path / "ckpt")
    export_official(cfg, w, d, variant="mxfp4", shards=3)
    cat = Catalog(d, cfg, "mxfp4", with_vision=False, with_engram=False)
    lazy = LazyOfficialWeights(cat)
    w13, sf13, w2, sf2 = lazy.expert_stack_fp4("layers.1", 4, 9, torch.device("cpu"))
    I = cfg.inter
    assert w13.shape == (5, 2 * I, cfg.hidden // 2) and w2.shape == (5, cfg.hidden, I // 2)
    eager = load_official(cat)
    for i, e in enumerate(range(4, 9)):
        raw1 = cat.read(f"layers.1.ffn.experts.{e}.w1.weight").view(torch.uint8)
        assert torch.equal(w13[i, :I], raw1)                                     # the checkpoint's bytes
        got13 = dequantize_expert_fp4(w13[i], sf13[i])
        assert torch.equal(got13[:I], eager[f"layers.1.ffn.experts.{e}.w1.weight"])
        assert torch.equal(got13[I:], eager[f"layers.1.ffn.experts.{e}.w3.weight"])
        assert torch.equal(dequantize_expert_fp4(w2[i], sf2[i]), eager[f"layers.1.ffn.experts.{e}.w2.weight"])
    s = torch.randint(0, 255, (3, 200, 16), dtype=torch.uint8)
    assert torch.equal(pack_sf_atoms_batched(s), torch.stack([pack_sf_atoms(x) for x in s]))
    # the engine takes this path for mxfp4 experts and ends with the same stacks
    ew = EngineWeights.from_fp32(cfg, lazy, 0, 1, torch.device("cpu"), expert_dtype="mxfp4")
    assert torch.equal(ew.layers[1].w13[4:9], w13) and torch.equal(ew.layers[1].w13_sf[4:9], sf13)
    assert lazy.expert_stack_fp4("layers.1", 0, 2, torch.device("cpu")) is not None
    nv = str(tmp_path / "nv")
    export_official(cfg, w, nv, variant="nvfp4", shards=2)
    other = LazyOfficialWeights(Catalog(nv, cfg, "nvfp4", with_vision=False, with_engram=False))
    assert other.expert_stack_fp4("layers.1", 0, 2, torch.device("cpu")) is None     # another expert format


def test_full_size_layer_loads_from_a_sparse_checkpoint(tmp_path):
    """One layer of the release model at its real tensor shapes (384 experts of 4608 x 5120 + 5120 x 2304 FP4 values, FP8
    dense projections, the 129280-row embedding and head), stored as a sparse file: the catalog validates all 2337
    tensors and rank 0 of 8 streams its shard into engine tensors - expert payloads byte for byte - in seconds."""
    import dataclasses
    import time
    from ds41rt_b200.loader.official import load_engine_weights
    cfg = dataclasses.replace(ModelConfig.flash(1), dspark=None, engram=None)
    want = expected_tensors(cfg, "mxfp4", False, False)
    size = {"BF16": 2, "F32": 4, "F8_E4M3": 1, "F8_E8M0": 1, "I8": 1, "U8": 1}
    hdr, cur = {}, 0
    for name, (dt, shape) in want.items():
        nb = size[dt]
        for s in shape:
            nb *= s
        hdr[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [cur, cur + nb]}
        cur += nb
    d = str(tmp_path)
    fname = "model-00001-of-00001.safetensors"
    _raw(os.path.join(d, fname), hdr, cur)                       # header + a hole of `cur` bytes
    json.dump({"metadata": {}, "weight_map": {n: fname for n in want}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    assert cur > 9 * (1 << 30) and os.stat(os.path.join(d, fname)).st_blocks * 512 < (64 << 20)
    t0 = time.time()
    ew = load_engine_weights(d, cfg, 0, 8, torch.device("cpu"), variant="mxfp4", expert_dtype="mxfp4")
    took = time.time() - t0
    lw = ew.layers[0]
    assert lw.w13.shape == (48, 4608, 2560) and lw.w13.dtype == torch.uint8          # 48 experts per rank, E2M1 pairs
    assert lw.w2.shape == (48, 5120, 1152) and lw.w13_sf.shape == (48, 36, 40, 512)
    assert ew.head.shape[0] == 129280 // 8
    print(f"one full-size layer, rank 0 of 8: {took:.1f} s")
    assert took < 120


def test_offline_conversion_to_the_nvfp4_variant_resumes_and_validates(tmp_path):
    """mxfp4 checkpoint -> NVFP4 variant shard by shard: experts re-quantised by the reference recipe, everything else
    byte for byte, an interrupted run continues from its receipts, and the result opens as a strict nvfp4 catalog."""
    from ds41rt_b200.loader.convert import convert_checkpoint
    from ds41rt_b200.ops import quant_ref as Q
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=2)
    src, dst = str(tmp_path / "src"), str(tmp_path / "dst")
    export_official(cfg, w, src, variant="mxfp4", shards=4)
    part = convert_checkpoint(src, dst, cfg, with_vision=False, with_engram=False, stop_after_shards=2)
    assert part["complete"] is False and part["written"] == 2
    assert not os.path.exists(os.path.join(dst, "model.safetensors.index.json"))
    full = convert_checkpoint(src, dst, cfg, with_vision=False, with_engram=False, link_unchanged=True)
    assert full["complete"] and full["already_done"] == 2 and full["written"] == 2
    again = convert_checkpoint(src, dst, cfg, with_vision=False, with_engram=False)
    assert again["already_done"] == 4 and again["written"] == 0
    a = Catalog(src, cfg, "mxfp4", with_vision=False, with_engram=False)
    b = Catalog(dst, cfg, "nvfp4", with_vision=False, with_engram=False)
    n_exp = sum(1 for n in a.expected if ".ffn.experts." in n and n.endswith(".weight"))
    assert part["expert_matrices"] + full["expert_matrices"] == n_exp
    name = "layers.1.ffn.experts.5.w1"
    vals = Q.dequant_mxfp4(a.read(name + ".weight").view(torch.uint8), a.read(name + ".scale").view(torch.uint8), 32)
    q, bs, gs = Q.quant_nvfp4(vals)
    assert torch.equal(b.read(name + ".weight").view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(b.read(name + ".weight_scale").view(torch.uint8), bs.view(torch.uint8))
    assert float(b.read(name + ".weight_scale_2")) == float(gs) and float(b.read(name + ".input_scale")) == 1.0
    back = Q.dequant_nvfp4(b.read(name + ".weight").view(torch.uint8), b.read(name + ".weight_scale"),
                           b.read(name + ".weight_scale_2").float())
    assert float((back - vals).norm() / vals.norm()) < 0.1     # FP4 codes re-rounded onto a finer scale grid
    for n in ("embed.weight", "layers.0.attn.wq_a.weight", "layers.0.attn.wq_a.scale", "norm.weight"):
        assert torch.equal(a.read(n).view(torch.uint8), b.read(n).view(torch.uint8)), n
    eager = load_official(b)
    ref = w[name + ".weight"]
    assert float((eager[name + ".weight"] - ref).abs().max()) < 0.3 * float(ref.abs().max())


def test_checkpoint_audit_reads_headers_only_and_names_what_is_inconsistent(tmp_path):
    """The header-level audit: identity digests that do not depend on where the checkpoint lies, catalog agreement, and
    a named error for an index that disagrees with the shards."""
    import json
    import shutil
    from ds41rt_b200.loader.audit import AuditError, audit, main
    cfg = ModelConfig.tiny()
    src = str(tmp_path / "src")
    export_official(cfg, init_weights(cfg, seed=2), src, variant="mxfp4", shards=3)
    rep = audit(src, payload_hashes=True, cfg=cfg, variant="mxfp4", with_vision=False, with_engram=False)
    assert rep["catalog"]["ok"] and len(rep["shards"]) == 3 and rep["tensors"] == sum(s["tensors"] for s in rep["shards"])
    assert rep["shard_bytes"] > sum(rep["bytes_by_dtype"].values()) > 0 and "I8" in rep["bytes_by_dtype"]
    assert all(len(s["file_sha256"]) == 64 for s in rep["shards"])
    copy = str(tmp_path / "elsewhere")
    shutil.copytree(src, copy)
    again = audit(copy)
    assert again["headers_sha256"] == rep["headers_sha256"] and again["index_sha256"] == rep["index_sha256"]
    assert "file_sha256" not in again["shards"][0] and "catalog" not in again
    assert audit(src, cfg=cfg, variant="nvfp4", with_vision=False, with_engram=False)["catalog"]["ok"] is False
    assert main([src, "--model", "tiny", "--no-vision", "--no-engram"]) == 0
    # an index that points a tensor at another shard, names a tensor nobody stores, or leaves the directory
    idx_path = os.path.join(copy, "model.safetensors.index.json")
    idx = json.load(open(idx_path))
    names = sorted(idx["weight_map"])
    shards = sorted(set(idx["weight_map"].values()))
    bad = json.loads(json.dumps(idx))
    bad["weight_map"][names[0]] = [s for s in shards if s != idx["weight_map"][names[0]]][0]
    json.dump(bad, open(idx_path, "w"))
    with pytest.raises(AuditError, match="the index says"):
        audit(copy)
    bad = json.loads(json.dumps(idx))
    bad["weight_map"]["ghost.weight"] = shards[0]
    json.dump(bad, open(idx_path, "w"))
    with pytest.raises(AuditError, match="in no shard"):
        audit(copy)
    bad = json.loads(json.dumps(idx))
    bad["weight_map"][names[0]] = "../" + shards[0]
    json.dump(bad, open(idx_path, "w"))
    with pytest.raises(AuditError, match="plain file name"):
        audit(copy)
    json.dump(idx, open(idx_path, "w"))
    with open(os.path.join(copy, shards[0]), "ab") as f:                        # trailing bytes: the payload no longer tiles
        f.write(b"\0" * 16)
    with pytest.raises(AuditError, match="trailing bytes"):
        audit(copy)
    assert main([copy]) == 1
