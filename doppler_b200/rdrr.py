"""RDRR artifact reader: manifest.json + shard_*.bin -> packed Q4_K weights in device memory.

Host mirror of the reference's artifact loading for the dense Q4_K decoder this library runs:

* manifest parsing and validation   src/formats/rdrr/parsing.js:29-80, validation.js:250-450
  (same normalisation of shard entries, same error strings, errors collected and raised together)
* tensor locations                  src/formats/rdrr/parsing.js:82-150 (``shard``/``shardIndex``,
  ``offset``, ``size``, optional ``spans`` for tensors that cross shard files)
* Q4_K upload                       src/loader/tensors/tensor-loader.js:540-558 (``loadQ4KFused``:
  the packed blocks are copied as they are; dtype ``Q4_K_M``, layout ``row``, shape ``[N, K]``,
  ``size == N * ceil(K/256) * 144``)

Only what the quantized-inference path needs is read: the decoder weights of a dense
Qwen3-style model (Q4_K_M projections, F16/F32/BF16 norms, F16 embedding, tied or separate LM
head).  Anything the path does not implement (MoE, sliding windows, softcapping, weight-offset
norms, column layout, non-Q4_K projections) is refused with a message naming the field instead of
being loaded wrongly.  ``write_artifact`` produces the same on-disk layout from in-memory weights;
the tests use it for round trips, and it is handy for exporting synthetic models.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Optional

import numpy as np

RDRR_VERSION = 1
Q4K_BLOCK_BYTES = 144
QK_K = 256
DEFAULT_SHARD_SIZE = 64 * 1024 * 1024  # the converter's shard size (manifest ``shards[i].size``)


class RdrrError(Exception):
    pass


# ---------------------------------------------------------------------------------------------
# manifest
# ---------------------------------------------------------------------------------------------
def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def validate_manifest(m: dict) -> List[str]:
    """Validation rules of src/formats/rdrr/validation.js that concern text decoders."""
    errors: List[str] = []
    version = m.get("version")
    if isinstance(version, str):
        try:
            version = float(version)
        except ValueError:
            version = None
    if not _is_num(version) or version != version or version < 1:
        errors.append(f"Invalid version: {m.get('version')}")
    for field in ("modelId", "modelType", "quantization"):
        if not m.get(field) or not isinstance(m.get(field), str):
            errors.append(f"Missing or invalid {field} field")
    if not isinstance(m.get("inference"), dict):
        errors.append("Missing or invalid inference field")
    if not m.get("hashAlgorithm"):
        errors.append("Missing or invalid hashAlgorithm")
    elif m["hashAlgorithm"] not in ("sha256", "blake3"):
        errors.append(f"Invalid hashAlgorithm: {m['hashAlgorithm']}")
    special = m.get("modelType") in ("diffusion", "energy", "embedding")
    eos = m.get("eos_token_id")
    if not special and "eos_token_id" not in m:
        errors.append("Missing eos_token_id")
    elif eos is not None:
        if isinstance(eos, list):
            if not eos or any(not _is_num(t) for t in eos):
                errors.append("Invalid eos_token_id array")
        elif not _is_num(eos):
            errors.append("Invalid eos_token_id")
    arch = m.get("architecture")
    if not special:
        if isinstance(arch, dict):
            for field in ("numLayers", "hiddenSize", "intermediateSize", "numAttentionHeads", "numKeyValueHeads", "headDim",
                          "vocabSize", "maxSeqLen"):
                v = arch.get(field)
                if not _is_num(v) or v <= 0:
                    errors.append(f"Invalid architecture.{field}")
        elif not arch:
            errors.append("Missing architecture field")
    if not m.get("tensorsFile") and not isinstance(m.get("tensors"), dict):
        errors.append("Missing tensorsFile and tensors - one is required")
    if isinstance(m.get("tensors"), dict):
        for name, loc in m["tensors"].items():
            if not isinstance(loc, dict) or not isinstance(loc.get("role"), str):
                errors.append(f'Tensor "{name}" missing role')
    shards = m.get("shards")
    if not isinstance(shards, list) or not shards:
        errors.append("Missing or empty shards array")
    else:
        expected = 0
        for i, sh in enumerate(shards):
            if sh.get("index") != i:
                errors.append(f"Shard {i} has incorrect index: {sh.get('index')}")
            if not _is_num(sh.get("size")) or sh["size"] <= 0:
                errors.append(f"Shard {i} has invalid size")
            h = sh.get("hash")
            if not h or not isinstance(h, str) or len(h) != 64:
                errors.append(f"Shard {i} has invalid hash")
            if not sh.get("filename") or not isinstance(sh.get("filename"), str):
                errors.append(f"Shard {i} has invalid filename")
            if sh.get("offset") != expected:
                errors.append(f"Shard {i} has incorrect offset: expected {expected}, got {sh.get('offset')}")
            expected += sh["size"] if _is_num(sh.get("size")) else 0
        if m.get("totalSize") != expected:
            errors.append(f"totalSize mismatch: declared {m.get('totalSize')}, calculated {expected}")
    return errors


def parse_manifest(text: str) -> dict:
    """parseManifest (src/formats/rdrr/parsing.js:29): JSON, shard normalisation, validation."""
    try:
        m = json.loads(text)
    except json.JSONDecodeError as e:
        raise RdrrError(f"Failed to parse manifest JSON: {e}") from None
    if not isinstance(m, dict):
        raise RdrrError("Failed to parse manifest JSON: not an object")
    if isinstance(m.get("shards"), list):
        offset, norm = 0, []
        algo = str(m.get("hashAlgorithm") or "").strip().lower()
        for i, sh in enumerate(m["shards"]):
            sh = sh if isinstance(sh, dict) else {}
            h = (sh.get("blake3") or sh.get("hash") or "") if algo == "blake3" else (sh.get("hash") or sh.get("blake3") or "")
            size = sh.get("size")
            norm.append({"index": sh.get("index", i), "filename": sh.get("filename") or sh.get("fileName") or "", "size": size,
                         "hash": h, "offset": sh.get("offset", offset), "hashAlgorithm": sh.get("hashAlgorithm")})
            offset += size if _is_num(size) else 0
        m["shards"] = norm
    errors = validate_manifest(m)
    if errors:
        raise RdrrError("Invalid manifest:\n  - " + "\n  - ".join(errors))
    return m


def parse_tensor_map(tensors: dict) -> Dict[str, dict]:
    """parseTensorMap (src/formats/rdrr/parsing.js:82): every tensor ends up with a ``spans`` list."""
    out: Dict[str, dict] = {}
    for name, loc in tensors.items():
        if not isinstance(loc.get("shape"), list):
            raise RdrrError(f"Tensor '{name}' missing shape")
        if not isinstance(loc.get("role"), str):
            raise RdrrError(f"Tensor '{name}' missing role")
        if not _is_num(loc.get("size")):
            raise RdrrError(f"Tensor '{name}' missing size")
        spans = None
        if "spans" in loc and loc["spans"] is not None:
            if not isinstance(loc["spans"], list):
                raise RdrrError(f"Tensor '{name}' has invalid spans array")
            spans = []
            for i, sp in enumerate(loc["spans"]):
                sp = sp if isinstance(sp, dict) else {}
                si = sp.get("shardIndex") if _is_num(sp.get("shardIndex")) else sp.get("shard")
                if not _is_num(si):
                    raise RdrrError(f"Tensor '{name}' span[{i}] missing shard index")
                if not _is_num(sp.get("offset")):
                    raise RdrrError(f"Tensor '{name}' span[{i}] missing offset")
                if not _is_num(sp.get("size")):
                    raise RdrrError(f"Tensor '{name}' span[{i}] missing size")
                spans.append({"shardIndex": int(si), "offset": int(sp["offset"]), "size": int(sp["size"])})
        else:
            si = loc.get("shardIndex") if _is_num(loc.get("shardIndex")) else loc.get("shard")
            if not _is_num(si):
                raise RdrrError(f"Tensor '{name}' missing shard index")
            if not _is_num(loc.get("offset")):
                raise RdrrError(f"Tensor '{name}' missing offset")
            spans = [{"shardIndex": int(si), "offset": int(loc["offset"]), "size": int(loc["size"])}]
        if sum(s["size"] for s in spans) != int(loc["size"]):
            raise RdrrError(f"Tensor '{name}' spans cover {sum(s['size'] for s in spans)} bytes, size says {loc['size']}")
        out[name] = dict(loc, spans=spans, size=int(loc["size"]))
    return out


# ---------------------------------------------------------------------------------------------
# artifact directory
# ---------------------------------------------------------------------------------------------
class RdrrArtifact:
    """A directory holding ``manifest.json`` and the shard files it names."""

    def __init__(self, path: str):
        self.path = path
        mpath = os.path.join(path, "manifest.json")
        if not os.path.isfile(mpath):
            raise RdrrError(f"no manifest.json in {path}")
        with open(mpath, "r", encoding="utf-8") as f:
            self.manifest = parse_manifest(f.read())
        if isinstance(self.manifest.get("tensors"), dict):
            raw = self.manifest["tensors"]
        else:
            tpath = os.path.join(path, self.manifest["tensorsFile"])
            if not os.path.isfile(tpath):
                raise RdrrError(f"tensorsFile '{self.manifest['tensorsFile']}' not found in {path}")
            with open(tpath, "r", encoding="utf-8") as f:
                raw = json.load(f)
        self.tensors = parse_tensor_map(raw)
        self._maps: Dict[int, np.memmap] = {}

    def _shard(self, index: int) -> np.memmap:
        shards = self.manifest["shards"]
        if index < 0 or index >= len(shards):
            raise RdrrError(f"shard index {index} out of range (manifest has {len(shards)} shards)")
        if index not in self._maps:
            sh = shards[index]
            fpath = os.path.join(self.path, sh["filename"])
            if not os.path.isfile(fpath):
                raise RdrrError(f"shard file '{sh['filename']}' is missing")
            actual = os.path.getsize(fpath)
            if actual != sh["size"]:
                raise RdrrError(f"shard file '{sh['filename']}' has {actual} bytes, manifest says {sh['size']}")
            self._maps[index] = np.memmap(fpath, dtype=np.uint8, mode="r")
        return self._maps[index]

    def verify_shards(self) -> List[int]:
        """Check shard hashes.  sha256 is checked here; blake3 needs a library this environment does
        not have, so those shards are returned as unverified instead of being trusted silently."""
        unverified = []
        algo = self.manifest["hashAlgorithm"]
        for sh in self.manifest["shards"]:
            if (sh.get("hashAlgorithm") or algo) != "sha256":
                unverified.append(sh["index"])
                continue
            got = hashlib.sha256(self._shard(sh["index"]).tobytes()).hexdigest()
            if got != sh["hash"]:
                raise RdrrError(f"shard {sh['index']} hash mismatch: manifest {sh['hash']}, file {got}")
        return unverified

    def has(self, name: str) -> bool:
        return name in self.tensors

    def location(self, name: str) -> dict:
        if name not in self.tensors:
            raise RdrrError(f"tensor '{name}' is not in the manifest")
        return self.tensors[name]

    def read_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes, spans concatenated in order (uint8, a copy)."""
        loc = self.location(name)
        out = np.empty(loc["size"], np.uint8)
        pos = 0
        for sp in loc["spans"]:
            shard = self._shard(sp["shardIndex"])
            if sp["offset"] < 0 or sp["offset"] + sp["size"] > shard.size:
                raise RdrrError(f"tensor '{name}' span [{sp['offset']}, +{sp['size']}) runs past shard {sp['shardIndex']} ({shard.size} bytes)")
            out[pos:pos + sp["size"]] = shard[sp["offset"]:sp["offset"] + sp["size"]]
            pos += sp["size"]
        return out

    # -- typed reads ---------------------------------------------------------------------
    def read_q4k(self, name: str, n: int, k: int) -> np.ndarray:
        loc = self.location(name)
        dtype = str(loc.get("dtype", "")).upper()
        if dtype not in ("Q4_K_M", "Q4_K"):
            raise RdrrError(f"tensor '{name}' has dtype {loc.get('dtype')}, this path takes Q4_K_M projections only")
        if loc.get("layout", "row") not in ("row", None):
            raise RdrrError(f"tensor '{name}' has layout '{loc.get('layout')}', this path takes the row layout only")
        if list(loc["shape"]) != [n, k]:
            raise RdrrError(f"tensor '{name}' has shape {loc['shape']}, the architecture needs [{n}, {k}]")
        want = n * ((k + QK_K - 1) // QK_K) * Q4K_BLOCK_BYTES
        if loc["size"] != want:
            raise RdrrError(f"tensor '{name}' holds {loc['size']} bytes, a row-layout Q4_K [{n}, {k}] matrix holds {want}")
        return self.read_bytes(name)

    def read_float(self, name: str, count: Optional[int] = None) -> np.ndarray:
        """F32 / F16 / BF16 tensor widened to float32."""
        loc = self.location(name)
        raw = self.read_bytes(name)
        dtype = str(loc.get("dtype", "")).upper()
        if dtype == "F32":
            v = raw.view(np.float32).copy()
        elif dtype == "F16":
            v = raw.view(np.float16).astype(np.float32)
        elif dtype == "BF16":
            v = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            raise RdrrError(f"tensor '{name}' has dtype {loc.get('dtype')}, expected F32, F16 or BF16")
        if count is not None and v.size != count:
            raise RdrrError(f"tensor '{name}' has {v.size} elements, the architecture needs {count}")
        return v

    def read_f16_rows(self, name: str, rows: int, cols: int) -> np.ndarray:
        loc = self.location(name)
        if str(loc.get("dtype", "")).upper() != "F16":
            raise RdrrError(f"tensor '{name}' has dtype {loc.get('dtype')}, this path keeps the embedding / LM head in F16")
        if list(loc["shape"]) != [rows, cols]:
            raise RdrrError(f"tensor '{name}' has shape {loc['shape']}, the architecture needs [{rows}, {cols}]")
        return self.read_bytes(name).view(np.float16).reshape(rows, cols)


# ---------------------------------------------------------------------------------------------
# manifest -> decoder configuration
# ---------------------------------------------------------------------------------------------
_UNSUPPORTED_INFERENCE = (
    # (section, field, value that this path implements)
    ("attention", "attnLogitSoftcapping", None), ("attention", "slidingWindow", None), ("attention", "valueNorm", False),
    ("attention", "attentionBias", False), ("attention", "attentionOutputGate", False), ("attention", "causal", True),
    ("normalization", "rmsNormWeightOffset", False), ("normalization", "preFeedforwardNorm", False),
    ("normalization", "postFeedforwardNorm", False), ("ffn", "activation", "silu"), ("ffn", "gatedActivation", True),
    ("ffn", "branchMode", "dense"), ("ffn", "useDoubleWideMlp", False), ("ffn", "swigluLimit", None),
    ("rope", "ropeScalingType", None), ("rope", "partialRotaryFactor", None), ("rope", "mropeInterleaved", False),
    ("output", "finalLogitSoftcapping", None), ("output", "scaleEmbeddings", False), ("output", "embeddingTranspose", False),
)


def decoder_config(manifest: dict) -> dict:
    """Architecture + inference fields -> the configuration dict DecoderModel takes.  Fields whose
    value asks for behaviour outside this path raise instead of being ignored."""
    arch = manifest.get("architecture")
    if not isinstance(arch, dict):
        raise RdrrError("manifest.architecture must be an object to build a decoder")
    if manifest.get("moeConfig"):
        raise RdrrError("manifest.moeConfig is set: mixture-of-experts models are outside this path")
    inf = manifest["inference"]
    for section, field, ok in _UNSUPPORTED_INFERENCE:
        sec = inf.get(section) or {}
        if field in sec and sec[field] != ok:
            raise RdrrError(f"inference.{section}.{field} = {sec[field]!r} is outside this path (implemented: {ok!r})")
    att = inf.get("attention") or {}
    if att.get("queryKeyNorm") is not True:
        raise RdrrError("inference.attention.queryKeyNorm must be true (per-head q/k RMSNorm is part of this decoder)")
    qpas = att.get("queryPreAttnScalar")
    if qpas is not None and qpas != arch["headDim"]:
        raise RdrrError(f"inference.attention.queryPreAttnScalar = {qpas} differs from headDim {arch['headDim']}: outside this path")
    norm = inf.get("normalization") or {}
    rope = inf.get("rope") or {}
    out = inf.get("output") or {}
    theta = rope.get("ropeTheta") or arch.get("ropeTheta")
    if not theta:
        raise RdrrError("inference.rope.ropeTheta is missing")
    if norm.get("rmsNormEps") is None:
        raise RdrrError("inference.normalization.rmsNormEps is missing")
    return {"n_layers": int(arch["numLayers"]), "hidden": int(arch["hiddenSize"]), "n_heads": int(arch["numAttentionHeads"]),
            "n_kv_heads": int(arch["numKeyValueHeads"]), "head_dim": int(arch["headDim"]), "inter": int(arch["intermediateSize"]),
            "vocab": int(arch["vocabSize"]), "eps": float(norm["rmsNormEps"]), "rope_theta": float(theta),
            "tie_word_embeddings": bool(out.get("tieWordEmbeddings", False)), "max_seq_len": int(arch["maxSeqLen"])}


_LAYER_TENSORS = {  # DecoderModel weight name -> tensor name inside a layer
    "wq": "self_attn.q_proj.weight", "wk": "self_attn.k_proj.weight", "wv": "self_attn.v_proj.weight",
    "wo": "self_attn.o_proj.weight", "wgate": "mlp.gate_proj.weight", "wup": "mlp.up_proj.weight",
    "wdown": "mlp.down_proj.weight", "in_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight",
    "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight",
}


def _prefix(art: RdrrArtifact) -> str:
    for p in ("model.", ""):
        if art.has(p + "embed_tokens.weight"):
            return p
    raise RdrrError("neither 'model.embed_tokens.weight' nor 'embed_tokens.weight' is in the manifest")


def layer_shapes(cfg: dict) -> dict:
    h, d = cfg["hidden"], cfg["head_dim"]
    return {"wq": (cfg["n_heads"] * d, h), "wk": (cfg["n_kv_heads"] * d, h), "wv": (cfg["n_kv_heads"] * d, h),
            "wo": (h, cfg["n_heads"] * d), "wgate": (cfg["inter"], h), "wup": (cfg["inter"], h), "wdown": (h, cfg["inter"])}


def read_layer(art: RdrrArtifact, cfg: dict, layer: int, prefix: Optional[str] = None) -> dict:
    """One layer's weights in the form DecoderModel.load_layer / the oracle model take."""
    prefix = _prefix(art) if prefix is None else prefix
    shapes = layer_shapes(cfg)
    out = {}
    for wname, tname in _LAYER_TENSORS.items():
        full = f"{prefix}layers.{layer}.{tname}"
        if wname in shapes:
            out[wname] = art.read_q4k(full, *shapes[wname])
        elif wname in ("q_norm", "k_norm"):
            out[wname] = art.read_float(full, cfg["head_dim"])
        else:
            out[wname] = art.read_float(full, cfg["hidden"])
    return out


def read_model_weights(art: RdrrArtifact, cfg: Optional[dict] = None) -> dict:
    """All weights on the host (small models and tests; load_decoder streams layer by layer)."""
    cfg = cfg or decoder_config(art.manifest)
    prefix = _prefix(art)
    embed = art.read_f16_rows(prefix + "embed_tokens.weight", cfg["vocab"], cfg["hidden"])
    if cfg.get("tie_word_embeddings") or not art.has("lm_head.weight"):
        lm_head = embed
    else:
        lm_head = art.read_f16_rows("lm_head.weight", cfg["vocab"], cfg["hidden"])
    return {"layers": [read_layer(art, cfg, i, prefix) for i in range(cfg["n_layers"])], "embed": embed, "lm_head": lm_head,
            "final_norm": art.read_float(prefix + "norm.weight", cfg["hidden"])}


def load_decoder(device, path: str, max_seq: int, max_batch: int = 1, tp_rank: int = 0, tp_size: int = 1, chunk_rows: int = 16384):
    """Open an artifact directory and upload it: the packed Q4_K bytes go to device memory as
    they are (loadQ4KFused), norms are widened to f32, the LM head is the embedding when tied.
    Under tensor parallelism every rank reads the whole tensor and the library keeps its slice."""
    from .model import DecoderModel  # needs the CUDA library; the reader itself does not

    art = RdrrArtifact(path)
    cfg = decoder_config(art.manifest)
    if max_seq > cfg["max_seq_len"]:
        raise RdrrError(f"max_seq {max_seq} exceeds the model's maxSeqLen {cfg['max_seq_len']}")
    prefix = _prefix(art)
    model = DecoderModel(device, cfg, max_seq, max_batch, tp_rank, tp_size)
    try:
        for i in range(cfg["n_layers"]):
            model.load_layer(i, read_layer(art, cfg, i, prefix))
        embed = art.read_f16_rows(prefix + "embed_tokens.weight", cfg["vocab"], cfg["hidden"])
        tied = cfg.get("tie_word_embeddings") or not art.has("lm_head.weight")
        head = embed if tied else art.read_f16_rows("lm_head.weight", cfg["vocab"], cfg["hidden"])
        shard = cfg["vocab"] // tp_size
        for r0 in range(0, cfg["vocab"], chunk_rows):
            rows = min(chunk_rows, cfg["vocab"] - r0)
            model.load_embed(embed[r0:r0 + rows], r0)
            lo, hi = max(r0, shard * tp_rank), min(r0 + rows, shard * (tp_rank + 1))
            if hi > lo:
                model.load_lm_head(head[lo:hi], lo)
        model.load_final_norm(art.read_float(prefix + "norm.weight", cfg["hidden"]))
    except Exception:
        model.destroy()
        raise
    return model


# ---------------------------------------------------------------------------------------------
# writer
# ---------------------------------------------------------------------------------------------
def write_artifact(path: str, cfg: dict, weights: dict, model_id: str = "synthetic-q4k", shard_size: int = DEFAULT_SHARD_SIZE,
                   prefix: str = "model.", norm_dtype: str = "F16", tie_word_embeddings: Optional[bool] = None) -> dict:
    """Write ``weights`` (the dict read_model_weights returns) as manifest.json + shard_NNNNN.bin.
    Tensors are packed back to back and cut at shard boundaries, so large tensors get ``spans``."""
    os.makedirs(path, exist_ok=True)
    tied = (weights["lm_head"] is weights["embed"]) if tie_word_embeddings is None else tie_word_embeddings
    items = []  # (name, bytes, shape, dtype, role, group, layout)

    def norm_bytes(w):
        w = np.asarray(w, np.float32)
        return (w.astype(np.float16) if norm_dtype == "F16" else w).tobytes(), norm_dtype

    items.append((prefix + "embed_tokens.weight", np.ascontiguousarray(weights["embed"], np.float16).tobytes(),
                  [cfg["vocab"], cfg["hidden"]], "F16", "embedding", "embed", None))
    shapes = layer_shapes(cfg)
    for i, lw in enumerate(weights["layers"]):
        for wname, tname in sorted(_LAYER_TENSORS.items(), key=lambda kv: kv[1]):
            full = f"{prefix}layers.{i}.{tname}"
            if wname in shapes:
                items.append((full, np.ascontiguousarray(lw[wname], np.uint8).tobytes(), list(shapes[wname]), "Q4_K_M", "matmul",
                              f"layer.{i}", "row"))
            else:
                b, dt = norm_bytes(lw[wname])
                items.append((full, b, [int(np.asarray(lw[wname]).size)], dt, "norm", f"layer.{i}", None))
    b, dt = norm_bytes(weights["final_norm"])
    items.append((prefix + "norm.weight", b, [cfg["hidden"]], dt, "norm", "head", None))
    if not tied:
        items.append(("lm_head.weight", np.ascontiguousarray(weights["lm_head"], np.float16).tobytes(), [cfg["vocab"], cfg["hidden"]],
                      "F16", "lm_head", "head", None))

    tensors, shards = {}, []
    cur = bytearray()

    def flush():
        idx = len(shards)
        fname = f"shard_{idx:05d}.bin"
        with open(os.path.join(path, fname), "wb") as f:
            f.write(cur)
        shards.append({"index": idx, "filename": fname, "size": len(cur), "hash": hashlib.sha256(bytes(cur)).hexdigest(),
                       "offset": sum(s["size"] for s in shards)})
        cur.clear()

    for name, data, shape, dtype, role, group, layout in items:
        spans, pos = [], 0
        while pos < len(data):
            if len(cur) == shard_size:
                flush()
            take = min(len(data) - pos, shard_size - len(cur))
            spans.append({"shardIndex": len(shards), "offset": len(cur), "size": take})
            cur += data[pos:pos + take]
            pos += take
        loc = {"size": len(data), "shape": shape, "dtype": dtype, "role": role, "group": group}
        if layout:
            loc["layout"] = layout
        if len(spans) == 1:
            loc.update({"shard": spans[0]["shardIndex"], "offset": spans[0]["offset"]})
        else:
            loc["spans"] = spans
        tensors[name] = loc
    if cur:
        flush()
    manifest = {
        "version": RDRR_VERSION, "modelId": model_id, "modelType": "transformer", "quantization": "Q4_K_M",
        "quantizationInfo": {"weights": "q4k", "embeddings": "f16", "compute": "f32", "layout": "row", "variantTag": "q4k-ehf16-af32"},
        "hashAlgorithm": "sha256", "eos_token_id": 0,
        "architecture": {"numLayers": cfg["n_layers"], "hiddenSize": cfg["hidden"], "intermediateSize": cfg["inter"],
                         "numAttentionHeads": cfg["n_heads"], "numKeyValueHeads": cfg["n_kv_heads"], "headDim": cfg["head_dim"],
                         "vocabSize": cfg["vocab"], "maxSeqLen": int(cfg.get("max_seq_len", 40960)),
                         "ropeTheta": cfg.get("rope_theta", 1e6)},
        "inference": {
            "schema": "doppler.execution/v1",
            "attention": {"queryPreAttnScalar": cfg["head_dim"], "attnLogitSoftcapping": None, "slidingWindow": None,
                          "queryKeyNorm": True, "valueNorm": False, "causal": True, "attentionBias": False,
                          "attentionOutputGate": False},
            "normalization": {"rmsNormEps": cfg.get("eps", 1e-6), "rmsNormWeightOffset": False, "postAttentionNorm": True,
                              "preFeedforwardNorm": False, "postFeedforwardNorm": False},
            "ffn": {"activation": "silu", "gatedActivation": True, "branchMode": "dense", "useDoubleWideMlp": False,
                    "swigluLimit": None},
            "rope": {"ropeTheta": cfg.get("rope_theta", 1e6), "ropeScalingType": None, "ropeScalingFactor": 1,
                     "partialRotaryFactor": None, "mropeInterleaved": False},
            "output": {"finalLogitSoftcapping": None, "tieWordEmbeddings": bool(tied), "scaleEmbeddings": False,
                       "embeddingTranspose": False},
        },
        "shards": shards, "tensors": tensors, "totalSize": sum(s["size"] for s in shards),
    }
    with open(os.path.join(path, "manifest.json"), "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=1)
    return manifest
