"""RDRR artifact reader (doppler_b200/rdrr.py): manifest rules of src/formats/rdrr/validation.js,
tensor spans across shard files, and the round trip artifact -> weights -> tokens."""
import copy
import json
import os

import numpy as np
import pytest

from doppler_b200 import rdrr, synthetic
from model_util import gaussian_model_weights

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tiny():
    cfg = dict(synthetic.MODEL_CONFIGS["tiny"])
    return cfg, gaussian_model_weights(cfg, 77)


def _same_weights(a, b):
    for la, lb in zip(a["layers"], b["layers"]):
        for k in la:
            assert np.array_equal(np.asarray(la[k]).view(np.uint8), np.asarray(lb[k]).view(np.uint8)), k
    for k in ("embed", "lm_head", "final_norm"):
        assert np.array_equal(np.asarray(a[k]).view(np.uint8), np.asarray(b[k]).view(np.uint8)), k


def test_round_trip_with_spans(tmp_path):
    cfg, w = _tiny()
    m = rdrr.write_artifact(str(tmp_path), cfg, w, shard_size=100_000, norm_dtype="F32")
    assert len(m["shards"]) > 5 and all(s["size"] == 100_000 for s in m["shards"][:-1])
    assert any("spans" in t for t in m["tensors"].values())           # tensors cut at shard boundaries
    assert any("shard" in t for t in m["tensors"].values())           # and tensors inside one shard
    art = rdrr.RdrrArtifact(str(tmp_path))
    assert art.verify_shards() == []
    got_cfg = rdrr.decoder_config(art.manifest)
    for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "inter", "vocab"):
        assert got_cfg[k] == cfg[k]
    assert got_cfg["tie_word_embeddings"] is False
    _same_weights(rdrr.read_model_weights(art), w)
    # the Q4_K size rule of the reference: N * ceil(K/256) * 144 bytes, layout 'row'
    loc = art.location("model.layers.0.mlp.down_proj.weight")
    assert loc["dtype"] == "Q4_K_M" and loc["layout"] == "row" and loc["size"] == cfg["hidden"] * (cfg["inter"] // 256) * 144


def test_tied_embeddings_prefixless_names_and_f16_norms(tmp_path):
    cfg, w = _tiny()
    w = dict(w, lm_head=w["embed"])
    m = rdrr.write_artifact(str(tmp_path), cfg, w, prefix="", norm_dtype="F16")
    assert "lm_head.weight" not in m["tensors"] and "embed_tokens.weight" in m["tensors"]
    art = rdrr.RdrrArtifact(str(tmp_path))
    got = rdrr.read_model_weights(art)
    assert got["lm_head"] is got["embed"]
    exp = np.asarray(w["layers"][1]["q_norm"], np.float32).astype(np.float16).astype(np.float32)
    assert np.array_equal(got["layers"][1]["q_norm"], exp)


def _manifest(tmp_path):
    cfg, w = _tiny()
    rdrr.write_artifact(str(tmp_path), cfg, w)
    return json.load(open(os.path.join(str(tmp_path), "manifest.json")))


def test_manifest_validation_messages(tmp_path):
    good = _manifest(tmp_path)
    rdrr.parse_manifest(json.dumps(good))
    cases = [
        (lambda m: m.pop("modelId"), "Missing or invalid modelId field"),
        (lambda m: m.update(version=0), "Invalid version: 0"),
        (lambda m: m.update(hashAlgorithm="md5"), "Invalid hashAlgorithm: md5"),
        (lambda m: m.pop("inference"), "Missing or invalid inference field"),
        (lambda m: m.pop("eos_token_id"), "Missing eos_token_id"),
        (lambda m: m["architecture"].update(headDim=0), "Invalid architecture.headDim"),
        (lambda m: m.update(totalSize=m["totalSize"] + 1), "totalSize mismatch"),
        (lambda m: m["shards"][0].update(hash="abc"), "Shard 0 has invalid hash"),
        (lambda m: m["shards"][0].update(index=3), "Shard 0 has incorrect index: 3"),
        (lambda m: m.pop("tensors"), "Missing tensorsFile and tensors - one is required"),
        (lambda m: m.update(shards=[]), "Missing or empty shards array"),
    ]
    for mutate, msg in cases:
        m = copy.deepcopy(good)
        mutate(m)
        with pytest.raises(rdrr.RdrrError, match="Invalid manifest") as e:
            rdrr.parse_manifest(json.dumps(m))
        assert msg in str(e.value), (msg, str(e.value))
    with pytest.raises(rdrr.RdrrError, match="Failed to parse manifest JSON"):
        rdrr.parse_manifest("{not json")
    # several problems are reported together, as the reference does
    m = copy.deepcopy(good)
    m.pop("modelId"); m.pop("quantization")
    with pytest.raises(rdrr.RdrrError) as e:
        rdrr.parse_manifest(json.dumps(m))
    assert "modelId" in str(e.value) and "quantization" in str(e.value)
    # fileName spelling and missing offsets are normalised (parsing.js:55-70)
    m = copy.deepcopy(good)
    for sh in m["shards"]:
        sh["fileName"] = sh.pop("filename")
        sh.pop("offset")
    assert rdrr.parse_manifest(json.dumps(m))["shards"][0]["filename"] == "shard_00000.bin"


def test_tensor_map_errors():
    base = {"shape": [2], "role": "norm", "size": 4, "dtype": "F16"}
    with pytest.raises(rdrr.RdrrError, match="missing shard index"):
        rdrr.parse_tensor_map({"t": dict(base, offset=0)})
    with pytest.raises(rdrr.RdrrError, match="missing offset"):
        rdrr.parse_tensor_map({"t": dict(base, shard=0)})
    with pytest.raises(rdrr.RdrrError, match="missing shape"):
        rdrr.parse_tensor_map({"t": {"role": "norm", "size": 4, "shard": 0, "offset": 0}})
    with pytest.raises(rdrr.RdrrError, match=r"span\[1\] missing size"):
        rdrr.parse_tensor_map({"t": dict(base, spans=[{"shardIndex": 0, "offset": 0, "size": 2}, {"shard": 1, "offset": 0}])})
    with pytest.raises(rdrr.RdrrError, match="spans cover"):
        rdrr.parse_tensor_map({"t": dict(base, spans=[{"shardIndex": 0, "offset": 0, "size": 2}])})
    ok = rdrr.parse_tensor_map({"t": dict(base, shardIndex=2, offset=8)})
    assert ok["t"]["spans"] == [{"shardIndex": 2, "offset": 8, "size": 4}]


def test_damaged_artifacts_are_refused(tmp_path):
    cfg, w = _tiny()
    d = str(tmp_path)
    rdrr.write_artifact(d, cfg, w, shard_size=1 << 20)
    # flipped byte: hash mismatch
    p = os.path.join(d, "shard_00001.bin")
    raw = bytearray(open(p, "rb").read())
    raw[100] ^= 0xFF
    open(p, "wb").write(raw)
    with pytest.raises(rdrr.RdrrError, match="shard 1 hash mismatch"):
        rdrr.RdrrArtifact(d).verify_shards()
    # truncated shard file
    open(p, "wb").write(raw[:-7])
    with pytest.raises(rdrr.RdrrError, match="manifest says"):
        rdrr.RdrrArtifact(d).verify_shards()
    os.remove(p)
    with pytest.raises(rdrr.RdrrError, match="is missing"):
        rdrr.read_model_weights(rdrr.RdrrArtifact(d))
    with pytest.raises(rdrr.RdrrError, match="no manifest.json"):
        rdrr.RdrrArtifact(os.path.join(d, "nowhere"))


def test_fields_outside_the_path_are_refused(tmp_path):
    good = _manifest(tmp_path)
    art = rdrr.RdrrArtifact(str(tmp_path))
    for section, field, value in [("attention", "slidingWindow", 512), ("attention", "attnLogitSoftcapping", 50.0),
                                  ("normalization", "rmsNormWeightOffset", True), ("ffn", "activation", "gelu"),
                                  ("output", "finalLogitSoftcapping", 30.0), ("attention", "queryKeyNorm", False)]:
        m = copy.deepcopy(good)
        m["inference"][section][field] = value
        with pytest.raises(rdrr.RdrrError, match=f"inference.{section}.{field}"):
            rdrr.decoder_config(m)
    m = copy.deepcopy(good)
    m["moeConfig"] = {"numExperts": 8, "numExpertsPerToken": 2}
    with pytest.raises(rdrr.RdrrError, match="moeConfig"):
        rdrr.decoder_config(m)
    # a projection that is not Q4_K_M, a column layout, a wrong byte count
    name = "model.layers.0.mlp.gate_proj.weight"
    n, k = rdrr.layer_shapes(_tiny()[0])["wgate"]
    for patch, msg in [({"dtype": "F16"}, "Q4_K_M projections only"), ({"layout": "col"}, "row layout only"),
                       ({"shape": [k, n]}, "architecture needs"), ]:
        saved = dict(art.tensors[name])
        art.tensors[name].update(patch)
        with pytest.raises(rdrr.RdrrError, match=msg):
            art.read_q4k(name, n, k)
        art.tensors[name] = saved
    with pytest.raises(rdrr.RdrrError, match="not in the manifest"):
        art.read_bytes("model.layers.99.mlp.up_proj.weight")


def test_oracle_runs_from_artifact(tmp_path):
    """Tokens from weights that went through an artifact equal the committed token fixture."""
    from oracle import oracle as O
    g = json.load(open(os.path.join(GOLDEN, "model_tokens.json")))
    cfg = dict(synthetic.MODEL_CONFIGS[g["config"]], max_seq=g["max_seq"])
    rdrr.write_artifact(str(tmp_path), cfg, gaussian_model_weights(cfg, g["seed"]), shard_size=8 << 20, norm_dtype="F32")
    art = rdrr.RdrrArtifact(str(tmp_path))
    cfg2 = dict(rdrr.decoder_config(art.manifest), max_seq=g["max_seq"])
    om = O.OracleModel(cfg2, rdrr.read_model_weights(art, cfg2))
    tok, _ = om.forward(np.array(g["prompt"], np.int32))
    toks = [tok]
    for _ in range(5):
        tok, _ = om.forward([tok])
        toks.append(tok)
    assert toks == g["tokens"][:6]


@pytest.mark.gpu
def test_load_decoder_from_artifact(dev, tmp_path):
    g = json.load(open(os.path.join(GOLDEN, "model_tokens.json")))
    cfg = dict(synthetic.MODEL_CONFIGS[g["config"]])
    rdrr.write_artifact(str(tmp_path), cfg, gaussian_model_weights(cfg, g["seed"]), shard_size=8 << 20, norm_dtype="F32")
    model = rdrr.load_decoder(dev, str(tmp_path), g["max_seq"])
    try:
        first = model.prefill(np.array(g["prompt"], np.int32))
        toks = [first] + [int(t) for t in model.decode([first], len(g["tokens"]) - 1)[:, 0]]
        assert toks == g["tokens"]
    finally:
        model.destroy()
    with pytest.raises(rdrr.RdrrError, match="exceeds the model's maxSeqLen"):
        rdrr.load_decoder(dev, str(tmp_path), 10 ** 9)


# ---- manifests the reference ships (models/local/<id>/manifest.json, committed gzip'd) ----------
def _reference_manifest(name):
    import gzip

    return gzip.open(os.path.join(GOLDEN, "manifest__" + name + ".json.gz"), "rt", encoding="utf-8").read()


def test_reference_manifest_of_the_0_6b_q4k_model_parses_to_the_baseline_shape():
    m = rdrr.parse_manifest(_reference_manifest("qwen-3-embedding-0-6b-q4k-ehf16-af32"))
    assert m["quantization"] == "Q4_K_M" and len(m["tensors"]) == 310
    cfg = rdrr.decoder_config(m)
    want = dict(n_layers=28, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, inter=3072, eps=1e-6, rope_theta=1e6)
    for k, v in want.items():
        assert cfg[k] == v, k
    assert cfg["tie_word_embeddings"] is True
    tmap = rdrr.parse_tensor_map(m["tensors"])
    H, I = cfg["hidden"], cfg["inter"]
    # packed Q4_K sizes follow N * ceil(K/256) * 144 (matmul-selection.js:230-233), row layout
    for name, (n, k) in {"q_proj": (2048, H), "k_proj": (1024, H), "o_proj": (H, 2048), "gate_proj": (I, H), "down_proj": (H, I)}.items():
        hits = [t for key, t in tmap.items() if key.endswith("layers.0." + ("self_attn." if "_proj" in name and name[0] in "qkvo" else "mlp.") + name + ".weight")]
        assert len(hits) == 1, name
        t = hits[0]
        assert t["dtype"] == "Q4_K_M" and t.get("layout", "row") == "row" and list(t["shape"]) == [n, k]
        assert t["size"] == n * ((k + 255) // 256) * 144


def test_reference_manifest_outside_the_path_is_refused_with_the_reason():
    m = rdrr.parse_manifest(_reference_manifest("qwen-3-5-0-8b-q4k-ehaf16"))
    assert len(m["tensors"]) == 489
    with pytest.raises(rdrr.RdrrError, match="attentionOutputGate"):
        rdrr.decoder_config(m)
