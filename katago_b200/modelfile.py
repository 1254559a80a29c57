"""KataGo model files: reader, writer, random-weight generator and blob serialiser.

Host-side logic only (numpy).  Mirrors the reference's model-file grammar
(cpp/neuralnet/desc.cpp:2280-2443 ModelDesc, :1566-1661 TrunkDesc, :545-555 / :624-638 /
:745-763 blocks, :1094-1172 attention, :1283-1304 FFN, :1914-2017 policy head, :2093-2188
value head; writer side python/export_model_pytorch.py:124-614).

A parsed model is a tree of plain dicts with numpy arrays in the SAME index order as the
reference's desc structs (conv weights [oc][ic][y][x], matmul weights [ic][oc]).  `to_blob`
flattens it into the record stream documented in include/kb_modelblob.h, which is what the
C ABI of the B200 library (and of the CPU oracle) consumes.
"""
from __future__ import annotations

import gzip
import io
import os
import struct
from typing import Any, Dict, List

import numpy as np

ACT_IDENTITY, ACT_RELU, ACT_MISH, ACT_SILU, ACT_MISH_SCALE8 = 0, 1, 2, 3, 12
_ACT_NAMES = {
    ACT_IDENTITY: "ACTIVATION_IDENTITY",
    ACT_RELU: "ACTIVATION_RELU",
    ACT_MISH: "ACTIVATION_MISH",
    ACT_SILU: "ACTIVATION_SILU",
}
_ACT_CODES = {v: k for k, v in _ACT_NAMES.items()}

TAG_MODEL, TAG_TRUNK, TAG_CONV, TAG_BN, TAG_MATMUL, TAG_MATBIAS, TAG_ACT = 1, 2, 3, 4, 5, 6, 7
TAG_BLOCK_ORDINARY, TAG_BLOCK_GPOOL, TAG_BLOCK_NESTED, TAG_BLOCK_ATTN, TAG_BLOCK_FFN = 10, 11, 12, 13, 14
TAG_ATTNBIAS = 17
TAG_METAENC = 22
TAG_RMSNORM, TAG_TRMSNORM, TAG_POLICYHEAD, TAG_VALUEHEAD, TAG_END = 15, 16, 20, 21, 99
BLOB_MAGIC = 0x314D424B

# model version -> (spatial features, global features); cpp/neuralnet/modelversion.cpp
_FEATURES = {3: (22, 14), 4: (22, 14), 5: (22, 14), 6: (13, 12), 7: (22, 16)}


def num_features(version: int):
    if version >= 8:
        return (22, 19)
    return _FEATURES[version]


# ----------------------------------------------------------------------------------------------
# Token reader over the reference's text / "@BIN@" format (desc.cpp:40-90)


class _Reader:
    def __init__(self, data: bytes, binary: bool):
        self.d = data
        self.p = 0
        self.binary = binary

    def token(self) -> str:
        d, p = self.d, self.p
        n = len(d)
        while p < n and d[p] in b" \t\r\n":
            p += 1
        s = p
        while p < n and d[p] not in b" \t\r\n":
            p += 1
        if s == p:
            raise ValueError("model file: unexpected end of file")
        self.p = p
        return d[s:p].decode("ascii")

    def int(self) -> int:
        return int(self.token())

    def float(self) -> float:
        return float(self.token())

    def floats(self, n: int, name: str) -> np.ndarray:
        if not self.binary:
            out = np.empty(n, dtype=np.float32)
            for i in range(n):
                out[i] = np.float32(float(self.token()))
        else:
            at = self.d.find(b"@", self.p)
            if at < 0 or at - self.p > 100 or self.d[at : at + 5] != b"@BIN@":
                raise ValueError(f"{name}: did not find expected header for binary float block")
            start = at + 5
            end = start + 4 * n
            if end > len(self.d):
                raise ValueError(f"{name}: did not find the expected number of floats in binary float block")
            out = np.frombuffer(self.d, dtype="<f4", count=n, offset=start).astype(np.float32)
            self.p = end
        if not np.all(np.isfinite(out)):
            raise ValueError(f"{name}: Nan or infinite neural net weight or parameter")
        return out


def _read_conv(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    ky, kx, ic, oc, dy, dx = (r.int() for _ in range(6))
    if ky <= 0 or kx <= 0 or ky % 2 != 1 or kx % 2 != 1:
        raise ValueError(f"{name}: convolution filter sizes must be odd and positive")
    if ic <= 0 or oc <= 0 or dy <= 0 or dx <= 0:
        raise ValueError(f"{name}: channels and dilations must be positive")
    w = r.floats(ky * kx * ic * oc, name).reshape(ky, kx, ic, oc)
    # file order y,x,ic,oc -> desc order oc,ic,y,x (desc.cpp:131-151)
    return dict(kind="conv", name=name, kY=ky, kX=kx, inC=ic, outC=oc, dilY=dy, dilX=dx,
                w=np.ascontiguousarray(w.transpose(3, 2, 0, 1)))


def _read_bn(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    c = r.int()
    eps = np.float32(r.float())
    has_scale, has_bias = r.int(), r.int()
    if c < 1 or not eps > 0:
        raise ValueError(f"{name}: bad channel count or epsilon")
    mean = r.floats(c, name)
    var = r.floats(c, name)
    scale = r.floats(c, name) if has_scale else np.ones(c, np.float32)
    bias = r.floats(c, name) if has_bias else np.zeros(c, np.float32)
    return dict(kind="bn", name=name, C=c, eps=eps, hasScale=has_scale, hasBias=has_bias,
                mean=mean, var=var, scale=scale, bias=bias)


def _read_act(r: _Reader, version: int) -> Dict[str, Any]:
    name = r.token()
    act = ACT_RELU
    if version >= 11:
        kind = r.token()
        if kind not in _ACT_CODES:
            raise ValueError(f"{name}: unknown activation {kind}")
        act = _ACT_CODES[kind]
    return dict(kind="act", name=name, act=act)


def _read_matmul(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    ic, oc = r.int(), r.int()
    if ic <= 0 or oc <= 0:
        raise ValueError(f"{name}: number of in and out channels must be positive")
    return dict(kind="matmul", name=name, inC=ic, outC=oc, w=r.floats(ic * oc, name).reshape(ic, oc))


def _read_matbias(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    c = r.int()
    if c <= 0:
        raise ValueError(f"{name}: number of channels must be positive")
    return dict(kind="matbias", name=name, C=c, w=r.floats(c, name))


def _read_trmsnorm(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    c = r.int()
    eps = np.float32(r.float())
    return dict(kind="trmsnorm", name=name, C=c, eps=eps, w=r.floats(c, name))


def _read_rmsnorm(r: _Reader) -> Dict[str, Any]:
    name = r.token()
    c = r.int()
    eps = np.float32(r.float())
    spatial, cgroup = r.int(), r.int()
    if cgroup != 0:
        raise ValueError(f"{name}: grouped spatial RMSNorm is not supported")
    return dict(kind="rmsnorm", name=name, C=c, eps=eps, spatial=spatial, gamma=r.floats(c, name), beta=r.floats(c, name))


def _read_blocks(r: _Reader, version: int, n: int) -> List[Dict[str, Any]]:
    blocks = []
    for _ in range(n):
        kind = r.token()
        if kind == "ordinary_block":
            b = dict(kind=kind, name=r.token())
            b["preBN"] = _read_bn(r); b["preAct"] = _read_act(r, version); b["conv1"] = _read_conv(r)
            b["midBN"] = _read_bn(r); b["midAct"] = _read_act(r, version); b["conv2"] = _read_conv(r)
        elif kind == "gpool_block":
            b = dict(kind=kind, name=r.token())
            b["preBN"] = _read_bn(r); b["preAct"] = _read_act(r, version)
            b["regularConv"] = _read_conv(r); b["gpoolConv"] = _read_conv(r)
            b["gpoolBN"] = _read_bn(r); b["gpoolAct"] = _read_act(r, version); b["gpoolToBias"] = _read_matmul(r)
            b["midBN"] = _read_bn(r); b["midAct"] = _read_act(r, version); b["finalConv"] = _read_conv(r)
        elif kind == "nested_bottleneck_block":
            b = dict(kind=kind, name=r.token())
            num_inner = r.int()
            b["preBN"] = _read_bn(r); b["preAct"] = _read_act(r, version); b["preConv"] = _read_conv(r)
            b["blocks"] = _read_blocks(r, version, num_inner)
            b["postBN"] = _read_bn(r); b["postAct"] = _read_act(r, version); b["postConv"] = _read_conv(r)
        elif kind == "transformer_attention_block":
            b = dict(kind=kind, name=r.token())
            b["heads"], b["kvHeads"], b["qDim"], b["vDim"] = r.int(), r.int(), r.int(), r.int()
            b["useRope"], b["learnableRope"] = r.int(), r.int()
            b["preLN"] = _read_trmsnorm(r)
            b["q"], b["k"], b["v"], b["out"] = _read_matmul(r), _read_matmul(r), _read_matmul(r), _read_matmul(r)
            if b["useRope"]:
                if b["learnableRope"]:
                    b["ropeName"] = r.token()
                    kvh, pairs, two = r.int(), r.int(), r.int()
                    if kvh != b["kvHeads"] or pairs != b["qDim"] // 2 or two != 2:
                        raise ValueError(f"{b['name']}: bad learnable rope header")
                    b["ropeFreqs"] = r.floats(kvh * pairs * 2, b["name"])
                else:
                    b["ropeName"] = r.token()
                    b["ropeTheta"] = np.float32(r.float())
        elif kind == "transformer_ffn_block":
            b = dict(kind=kind, name=r.token())
            b["C"], b["ffnC"], b["swiglu"] = r.int(), r.int(), r.int()
            b["preLN"] = _read_trmsnorm(r)
            b["linear1"] = _read_matmul(r)
            if b["swiglu"]:
                b["gate"] = _read_matmul(r)
            b["linear2"] = _read_matmul(r)
        else:
            raise ValueError(f"found unknown block kind: {kind}")
        blocks.append(b)
    return blocks


def parse_model_bytes(data: bytes, binary: bool) -> Dict[str, Any]:
    r = _Reader(data, binary)
    m: Dict[str, Any] = dict(name=r.token())
    v = m["version"] = r.int()
    if v < 3 or v > 17:
        raise ValueError(f"unsupported model version {v}")
    m["numInputChannels"], m["numInputGlobalChannels"] = r.int(), r.int()
    m["postProcess"] = [r.float() for _ in range(7)] if v >= 13 else None
    m["metaEncoderVersion"] = 0
    if v >= 15:
        m["metaEncoderVersion"] = r.int()
        for _ in range(7):
            if r.int() != 0:
                raise ValueError("unknown/unsupported model option")
    if m["metaEncoderVersion"] not in (0, 1):
        raise ValueError("unsupported SGF metadata encoder version")
    t: Dict[str, Any] = dict(name=r.token())
    t["numBlocks"], t["trunkC"], t["midC"], t["regularC"], t["dilatedC"], t["gpoolC"] = (r.int() for _ in range(6))
    t["normKind"] = 0
    if v >= 15:
        t["normKind"] = r.int()
        for _ in range(5):
            if r.int() != 0:
                raise ValueError("unknown/unsupported trunk option")
    t["initialConv"] = _read_conv(r)
    t["initialMatMul"] = _read_matmul(r)
    if m["metaEncoderVersion"] > 0:
        # SGFMetadataEncoderDesc, desc.cpp:1476-1522
        e: Dict[str, Any] = dict(name=r.token(), numInputMetaChannels=r.int())
        e["mul1"] = _read_matmul(r); e["bias1"] = _read_matbias(r); e["act1"] = _read_act(r, v)
        e["mul2"] = _read_matmul(r); e["bias2"] = _read_matbias(r); e["act2"] = _read_act(r, v)
        e["mul3"] = _read_matmul(r)
        t["metaEncoder"] = e
    t["blocks"] = _read_blocks(r, v, t["numBlocks"])
    if t["normKind"] == 0:
        t["tipBN"] = _read_bn(r)
    else:
        t["tipRMSNorm"] = _read_rmsnorm(r)
    t["tipAct"] = _read_act(r, v)
    m["trunk"] = t
    p: Dict[str, Any] = dict(name=r.token())
    if v >= 17:
        p["policyC"] = r.int()
        for _ in range(3):
            if r.int() != 0:
                raise ValueError("unknown/unsupported policy option")
    elif v == 16:
        p["policyC"] = 4
    elif v >= 12:
        p["policyC"] = 2
    else:
        p["policyC"] = 1
    p["p1Conv"], p["g1Conv"] = _read_conv(r), _read_conv(r)
    p["g1BN"], p["g1Act"] = _read_bn(r), _read_act(r, v)
    p["gpoolToBias"] = _read_matmul(r)
    p["p1BN"], p["p1Act"] = _read_bn(r), _read_act(r, v)
    p["p2Conv"] = _read_conv(r)
    p["passMul"] = _read_matmul(r)
    if v >= 15:
        p["passBias"], p["passAct"], p["passMul2"] = _read_matbias(r), _read_act(r, v), _read_matmul(r)
    m["policyHead"] = p
    h: Dict[str, Any] = dict(name=r.token())
    if v >= 17:
        for _ in range(3):
            if r.int() != 0:
                raise ValueError("unknown/unsupported value option")
    h["v1Conv"], h["v1BN"], h["v1Act"] = _read_conv(r), _read_bn(r), _read_act(r, v)
    h["v2Mul"], h["v2Bias"], h["v2Act"] = _read_matmul(r), _read_matbias(r), _read_act(r, v)
    h["v3Mul"], h["v3Bias"] = _read_matmul(r), _read_matbias(r)
    h["sv3Mul"], h["sv3Bias"] = _read_matmul(r), _read_matbias(r)
    h["ownConv"] = _read_conv(r)
    m["valueHead"] = h
    return m


def load_model_file(path: str) -> Dict[str, Any]:
    """Reads .bin.gz / .txt.gz / .bin / .txt model files (desc.cpp:2574-2636), and the extension file next to it
    (<path>.kbext, see model_ext_bytes) if there is one."""
    lower = path.lower()
    with open(path, "rb") as f:
        raw = f.read()
    if lower.endswith(".gz"):
        raw = gzip.decompress(raw)
    binary = not (lower.endswith(".txt.gz") or lower.endswith(".txt"))
    m = parse_model_bytes(raw, binary)
    if os.path.exists(path + EXT_SUFFIX):
        with open(path + EXT_SUFFIX, "rb") as f:
            attach_model_ext(m, f.read())
    return m


# ----------------------------------------------------------------------------------------------
# Extension file: weights the reference's model file format has no field for (katago_b200/host/model_ext.h gives the
# encoding and is the reader the backends use).  Today: the learned relative-position attention bias, by block name.

EXT_SUFFIX = ".kbext"
_EXT_MAGIC = b"KBMDLEXT"
_EXT_KIND_ATTNBIAS = 1


def _attention_blocks(blocks):
    for b in blocks:
        if b["kind"] == "transformer_attention_block":
            yield b
        elif b["kind"] == "nested_bottleneck_block":
            yield from _attention_blocks(b["blocks"])


def _ext_str(s: str) -> bytes:
    raw = s.encode("ascii")
    return struct.pack("<I", len(raw)) + raw + b"\0" * (-len(raw) % 4)


def model_ext_bytes(m: Dict[str, Any]):
    """The extension file's content for a model, or None if the model has nothing that needs one."""
    recs = []
    for b in _attention_blocks(m["trunk"]["blocks"]):
        if b.get("relBias") is None:
            continue
        rb = np.ascontiguousarray(b["relBias"], dtype="<f4")
        if rb.ndim != 3 or rb.shape[0] != b["heads"] or rb.shape[1] % 2 != 1 or rb.shape[2] % 2 != 1:
            raise ValueError(f"{b['name']}: a relative-position bias is [heads][2Y-1][2X-1]")
        payload = _ext_str(b["name"]) + struct.pack("<III", rb.shape[0], (rb.shape[1] + 1) // 2, (rb.shape[2] + 1) // 2) + rb.tobytes()
        recs.append(struct.pack("<II", _EXT_KIND_ATTNBIAS, len(payload)) + payload)
    if not recs:
        return None
    names = [b["name"] for b in _attention_blocks(m["trunk"]["blocks"])]
    if len(set(names)) != len(names):
        raise ValueError("attention blocks must have distinct names for the extension file to address them")
    return _EXT_MAGIC + struct.pack("<I", 1) + _ext_str(m["name"]) + struct.pack("<I", len(recs)) + b"".join(recs)


def attach_model_ext(m: Dict[str, Any], data: bytes) -> None:
    """Attaches the records of an extension file to the model tree; the same checks as the C++ reader."""
    pos = 0

    def take(n):
        nonlocal pos
        if pos + n > len(data):
            raise ValueError("model extension file is truncated")
        out = data[pos:pos + n]
        pos += n
        return out

    def u32():
        return struct.unpack("<I", take(4))[0]

    def string():
        n = u32()
        if n > 4096:
            raise ValueError("model extension file holds a malformed name")
        raw = take((n + 3) // 4 * 4)
        return raw[:n].decode("ascii")

    if take(8) != _EXT_MAGIC:
        raise ValueError("not a model extension file")
    version = u32()
    if version != 1:
        raise ValueError(f"model extension format version {version} is not supported (this reader knows 1)")
    name = string()
    if name != m["name"]:
        raise ValueError(f"model extension file written for model '{name}', but the model file holds '{m['name']}'")
    by_name = {b["name"]: b for b in _attention_blocks(m["trunk"]["blocks"])}
    seen = set()
    for _ in range(u32()):
        kind, nbytes = u32(), u32()
        end = pos + nbytes
        if nbytes % 4 or end > len(data):
            raise ValueError("model extension file: record runs past the end of the file")
        if kind != _EXT_KIND_ATTNBIAS:
            raise ValueError(f"model extension file: unknown record kind {kind}")
        block = string()
        heads, Y, X = u32(), u32(), u32()
        if not (1 <= heads <= 1024 and 1 <= Y <= 64 and 1 <= X <= 64):
            raise ValueError(f"model extension file: attention bias of block '{block}' has an invalid shape")
        n = heads * (2 * Y - 1) * (2 * X - 1)
        if pos + 4 * n != end:
            raise ValueError(f"model extension file: attention bias of block '{block}' does not match its record length")
        table = np.frombuffer(take(4 * n), dtype="<f4").reshape(heads, 2 * Y - 1, 2 * X - 1).astype(np.float32)
        if block not in by_name:
            raise ValueError(f"model extension file names a block the model does not have: '{block}'")
        if block in seen:
            raise ValueError(f"model extension file: two attention bias records for block '{block}'")
        if by_name[block]["heads"] != heads:
            raise ValueError(f"model extension file: attention bias of block '{block}' has {heads} heads, the block {by_name[block]['heads']}")
        seen.add(block)
        by_name[block]["relBias"] = table
    if pos != len(data):
        raise ValueError("model extension file: bytes after the last record")


# ----------------------------------------------------------------------------------------------
# Writer (binary "@BIN@" flavour, python/export_model_pytorch.py:162-168)


class _Writer:
    def __init__(self):
        self.b = io.BytesIO()

    def ln(self, *items):
        self.b.write((" ".join(str(x) for x in items) + "\n").encode("ascii"))

    def floats(self, arr):
        a = np.ascontiguousarray(arr, dtype="<f4")
        self.b.write(b"@BIN@" + a.tobytes() + b"\n")


def _write_conv(w: _Writer, c):
    w.ln(c["name"]); w.ln(c["kY"], c["kX"], c["inC"], c["outC"], c["dilY"], c["dilX"])
    w.floats(np.asarray(c["w"]).transpose(2, 3, 1, 0))  # oc,ic,y,x -> y,x,ic,oc


def _write_bn(w: _Writer, b):
    w.ln(b["name"]); w.ln(b["C"]); w.ln(repr(float(b["eps"]))); w.ln(1 if b["hasScale"] else 0, 1 if b["hasBias"] else 0)
    w.floats(b["mean"]); w.floats(b["var"])
    if b["hasScale"]:
        w.floats(b["scale"])
    if b["hasBias"]:
        w.floats(b["bias"])


def _write_act(w: _Writer, a, version):
    w.ln(a["name"])
    if version >= 11:
        w.ln(_ACT_NAMES[a["act"]])


def _write_matmul(w: _Writer, m):
    w.ln(m["name"]); w.ln(m["inC"], m["outC"]); w.floats(m["w"])


def _write_matbias(w: _Writer, m):
    w.ln(m["name"]); w.ln(m["C"]); w.floats(m["w"])


def _write_trmsnorm(w: _Writer, t):
    w.ln(t["name"]); w.ln(t["C"]); w.ln(repr(float(t["eps"]))); w.floats(t["w"])


def _write_blocks(w: _Writer, blocks, v):
    for b in blocks:
        w.ln(b["kind"]); w.ln(b["name"])
        k = b["kind"]
        if k == "ordinary_block":
            _write_bn(w, b["preBN"]); _write_act(w, b["preAct"], v); _write_conv(w, b["conv1"])
            _write_bn(w, b["midBN"]); _write_act(w, b["midAct"], v); _write_conv(w, b["conv2"])
        elif k == "gpool_block":
            _write_bn(w, b["preBN"]); _write_act(w, b["preAct"], v); _write_conv(w, b["regularConv"]); _write_conv(w, b["gpoolConv"])
            _write_bn(w, b["gpoolBN"]); _write_act(w, b["gpoolAct"], v); _write_matmul(w, b["gpoolToBias"])
            _write_bn(w, b["midBN"]); _write_act(w, b["midAct"], v); _write_conv(w, b["finalConv"])
        elif k == "nested_bottleneck_block":
            w.ln(len(b["blocks"]))
            _write_bn(w, b["preBN"]); _write_act(w, b["preAct"], v); _write_conv(w, b["preConv"])
            _write_blocks(w, b["blocks"], v)
            _write_bn(w, b["postBN"]); _write_act(w, b["postAct"], v); _write_conv(w, b["postConv"])
        elif k == "transformer_attention_block":
            # a relative-position bias has no field in this format: it travels in the extension file (model_ext_bytes)
            w.ln(b["heads"], b["kvHeads"], b["qDim"], b["vDim"], b["useRope"], b["learnableRope"])
            _write_trmsnorm(w, b["preLN"])
            for key in ("q", "k", "v", "out"):
                _write_matmul(w, b[key])
            if b["useRope"]:
                if b["learnableRope"]:
                    w.ln(b.get("ropeName", b["name"] + "/rope_freqs")); w.ln(b["kvHeads"], b["qDim"] // 2, 2); w.floats(b["ropeFreqs"])
                else:
                    w.ln(b.get("ropeName", b["name"] + "/rope_theta")); w.ln(repr(float(b["ropeTheta"])))
        elif k == "transformer_ffn_block":
            w.ln(b["C"], b["ffnC"], b["swiglu"])
            _write_trmsnorm(w, b["preLN"]); _write_matmul(w, b["linear1"])
            if b["swiglu"]:
                _write_matmul(w, b["gate"])
            _write_matmul(w, b["linear2"])
        else:
            raise ValueError(k)


def model_file_bytes(m: Dict[str, Any]) -> bytes:
    w = _Writer()
    v = m["version"]
    w.ln(m["name"]); w.ln(v); w.ln(m["numInputChannels"]); w.ln(m["numInputGlobalChannels"])
    if v >= 13:
        for x in m["postProcess"]:
            w.ln(repr(float(x)))
    if v >= 15:
        w.ln(m.get("metaEncoderVersion", 0))
        for _ in range(7):
            w.ln(0)
    t = m["trunk"]
    w.ln(t["name"]); w.ln(t["numBlocks"]); w.ln(t["trunkC"]); w.ln(t["midC"]); w.ln(t["regularC"]); w.ln(t["dilatedC"]); w.ln(t["gpoolC"])
    if v >= 15:
        w.ln(t["normKind"])
        for _ in range(5):
            w.ln(0)
    _write_conv(w, t["initialConv"]); _write_matmul(w, t["initialMatMul"])
    if m.get("metaEncoderVersion", 0) > 0:
        e = t["metaEncoder"]
        w.ln(e["name"]); w.ln(e["numInputMetaChannels"])
        _write_matmul(w, e["mul1"]); _write_matbias(w, e["bias1"]); _write_act(w, e["act1"], v)
        _write_matmul(w, e["mul2"]); _write_matbias(w, e["bias2"]); _write_act(w, e["act2"], v)
        _write_matmul(w, e["mul3"])
    _write_blocks(w, t["blocks"], v)
    if t["normKind"] == 0:
        _write_bn(w, t["tipBN"])
    else:
        r = t["tipRMSNorm"]
        w.ln(r["name"]); w.ln(r["C"]); w.ln(repr(float(r["eps"]))); w.ln(r["spatial"], 0); w.floats(r["gamma"]); w.floats(r["beta"])
    _write_act(w, t["tipAct"], v)
    p = m["policyHead"]
    w.ln(p["name"])
    if v >= 17:
        w.ln(p["policyC"])
        for _ in range(3):
            w.ln(0)
    _write_conv(w, p["p1Conv"]); _write_conv(w, p["g1Conv"]); _write_bn(w, p["g1BN"]); _write_act(w, p["g1Act"], v)
    _write_matmul(w, p["gpoolToBias"]); _write_bn(w, p["p1BN"]); _write_act(w, p["p1Act"], v); _write_conv(w, p["p2Conv"])
    _write_matmul(w, p["passMul"])
    if v >= 15:
        _write_matbias(w, p["passBias"]); _write_act(w, p["passAct"], v); _write_matmul(w, p["passMul2"])
    h = m["valueHead"]
    w.ln(h["name"])
    if v >= 17:
        for _ in range(3):
            w.ln(0)
    _write_conv(w, h["v1Conv"]); _write_bn(w, h["v1BN"]); _write_act(w, h["v1Act"], v)
    _write_matmul(w, h["v2Mul"]); _write_matbias(w, h["v2Bias"]); _write_act(w, h["v2Act"], v)
    _write_matmul(w, h["v3Mul"]); _write_matbias(w, h["v3Bias"]); _write_matmul(w, h["sv3Mul"]); _write_matbias(w, h["sv3Bias"])
    _write_conv(w, h["ownConv"])
    return w.b.getvalue()


def save_model_file(m: Dict[str, Any], path: str) -> None:
    """Writes the model file and, if the model holds weights the format has no field for (model_ext_bytes), the
    extension file <path>.kbext next to it; an extension file left over from another model is removed."""
    if not path.endswith(".bin.gz"):
        raise ValueError("model files are written in the .bin.gz flavour")
    with open(path, "wb") as f:
        f.write(gzip.compress(model_file_bytes(m), compresslevel=1, mtime=0))
    ext = model_ext_bytes(m)
    if ext is not None:
        with open(path + EXT_SUFFIX, "wb") as f:
            f.write(ext)
    elif os.path.exists(path + EXT_SUFFIX):
        os.remove(path + EXT_SUFFIX)


# ----------------------------------------------------------------------------------------------
# Blob serialiser (include/kb_modelblob.h)


class _Blob:
    def __init__(self):
        self.parts: List[bytes] = []
        self.words = 3

    def rec(self, tag: int, ints=(), floats=None):
        fl = np.zeros(0, "<f4") if floats is None else np.ascontiguousarray(floats, dtype="<f4").ravel()
        head = struct.pack(f"<II{len(ints)}iI", tag, len(ints), *[int(i) for i in ints], fl.size)
        self.parts.append(head)
        self.parts.append(fl.tobytes())
        self.words += 3 + len(ints) + fl.size

    def finish(self) -> bytes:
        return struct.pack("<III", BLOB_MAGIC, 1, self.words) + b"".join(self.parts)


def merged_bn(b):
    """desc.cpp:278-285 computeMerged, in fp32 like the reference."""
    scale = (b["scale"].astype(np.float32) / np.sqrt(b["var"].astype(np.float32) + np.float32(b["eps"]))).astype(np.float32)
    bias = (b["bias"].astype(np.float32) - scale * b["mean"].astype(np.float32)).astype(np.float32)
    return scale, bias


def _b_conv(o: _Blob, c):
    o.rec(TAG_CONV, (c["kY"], c["kX"], c["inC"], c["outC"], c["dilY"], c["dilX"]), c["w"])


def _b_bn(o: _Blob, b, act):
    s, bi = merged_bn(b)
    o.rec(TAG_BN, (b["C"], act), np.concatenate([s, bi]))


def _b_matmul(o: _Blob, m):
    o.rec(TAG_MATMUL, (m["inC"], m["outC"]), m["w"])


def _b_matbias(o: _Blob, m):
    o.rec(TAG_MATBIAS, (m["C"],), m["w"])


def _b_trms(o: _Blob, t):
    o.rec(TAG_TRMSNORM, (t["C"],), np.concatenate([[np.float32(t["eps"])], t["w"]]))


def _b_blocks(o: _Blob, blocks):
    for b in blocks:
        k = b["kind"]
        if k == "ordinary_block":
            o.rec(TAG_BLOCK_ORDINARY)
            _b_bn(o, b["preBN"], b["preAct"]["act"]); _b_conv(o, b["conv1"]); _b_bn(o, b["midBN"], b["midAct"]["act"]); _b_conv(o, b["conv2"])
        elif k == "gpool_block":
            o.rec(TAG_BLOCK_GPOOL)
            _b_bn(o, b["preBN"], b["preAct"]["act"]); _b_conv(o, b["regularConv"]); _b_conv(o, b["gpoolConv"])
            _b_bn(o, b["gpoolBN"], b["gpoolAct"]["act"]); _b_matmul(o, b["gpoolToBias"])
            _b_bn(o, b["midBN"], b["midAct"]["act"]); _b_conv(o, b["finalConv"])
        elif k == "nested_bottleneck_block":
            o.rec(TAG_BLOCK_NESTED, (len(b["blocks"]),))
            _b_bn(o, b["preBN"], b["preAct"]["act"]); _b_conv(o, b["preConv"])
            _b_blocks(o, b["blocks"])
            _b_bn(o, b["postBN"], b["postAct"]["act"]); _b_conv(o, b["postConv"])
        elif k == "transformer_attention_block":
            fl = None
            if b["useRope"]:
                fl = b["ropeFreqs"] if b["learnableRope"] else np.array([b["ropeTheta"]], np.float32)
            o.rec(TAG_BLOCK_ATTN, (b["heads"], b["kvHeads"], b["qDim"], b["vDim"], b["useRope"], b["learnableRope"]), fl)
            _b_trms(o, b["preLN"])
            for key in ("q", "k", "v", "out"):
                _b_matmul(o, b[key])
            if b.get("relBias") is not None:
                # learned relative-position bias [heads][2Y-1][2X-1]: an extension carried by the blob only
                rb = np.asarray(b["relBias"], np.float32)
                o.rec(TAG_ATTNBIAS, (rb.shape[0], (rb.shape[1] + 1) // 2, (rb.shape[2] + 1) // 2), rb.reshape(-1))
        elif k == "transformer_ffn_block":
            o.rec(TAG_BLOCK_FFN, (b["C"], b["ffnC"], b["swiglu"]))
            _b_trms(o, b["preLN"]); _b_matmul(o, b["linear1"])
            if b["swiglu"]:
                _b_matmul(o, b["gate"])
            _b_matmul(o, b["linear2"])
        else:
            raise ValueError(k)


def to_blob(m: Dict[str, Any]) -> bytes:
    o = _Blob()
    v = m["version"]
    p, h, t = m["policyHead"], m["valueHead"], m["trunk"]
    enc = t.get("metaEncoder") if m.get("metaEncoderVersion", 0) > 0 else None
    o.rec(TAG_MODEL, (v, m["numInputChannels"], m["numInputGlobalChannels"], enc["numInputMetaChannels"] if enc else 0, p["policyC"],
                      h["v3Mul"]["outC"], h["sv3Mul"]["outC"], h["ownConv"]["outC"]))
    o.rec(TAG_TRUNK, (t["numBlocks"], t["trunkC"], t["midC"], t["regularC"], t["gpoolC"], t["normKind"]))
    _b_conv(o, t["initialConv"]); _b_matmul(o, t["initialMatMul"])
    if enc:
        o.rec(TAG_METAENC, (m["metaEncoderVersion"], enc["numInputMetaChannels"]))
        _b_matmul(o, enc["mul1"]); _b_matbias(o, enc["bias1"]); o.rec(TAG_ACT, (enc["act1"]["act"],))
        _b_matmul(o, enc["mul2"]); _b_matbias(o, enc["bias2"]); o.rec(TAG_ACT, (enc["act2"]["act"],))
        _b_matmul(o, enc["mul3"])
    _b_blocks(o, t["blocks"])
    if t["normKind"] == 0:
        _b_bn(o, t["tipBN"], t["tipAct"]["act"])
    else:
        r = t["tipRMSNorm"]
        o.rec(TAG_RMSNORM, (r["C"], r["spatial"], t["tipAct"]["act"]), np.concatenate([[np.float32(r["eps"])], r["gamma"], r["beta"]]))
    has_pass_mlp = 1 if v >= 15 else 0
    o.rec(TAG_POLICYHEAD, (v, p["policyC"], has_pass_mlp))
    _b_conv(o, p["p1Conv"]); _b_conv(o, p["g1Conv"]); _b_bn(o, p["g1BN"], p["g1Act"]["act"]); _b_matmul(o, p["gpoolToBias"])
    _b_bn(o, p["p1BN"], p["p1Act"]["act"]); _b_conv(o, p["p2Conv"]); _b_matmul(o, p["passMul"])
    if has_pass_mlp:
        _b_matbias(o, p["passBias"]); o.rec(TAG_ACT, (p["passAct"]["act"],)); _b_matmul(o, p["passMul2"])
    o.rec(TAG_VALUEHEAD, (v,))
    _b_conv(o, h["v1Conv"]); _b_bn(o, h["v1BN"], h["v1Act"]["act"]); _b_matmul(o, h["v2Mul"]); _b_matbias(o, h["v2Bias"])
    o.rec(TAG_ACT, (h["v2Act"]["act"],)); _b_matmul(o, h["v3Mul"]); _b_matbias(o, h["v3Bias"])
    _b_matmul(o, h["sv3Mul"]); _b_matbias(o, h["sv3Bias"]); _b_conv(o, h["ownConv"])
    o.rec(TAG_END)
    return o.finish()


def layer_blob(layer: Dict[str, Any], act: int = ACT_IDENTITY) -> bytes:
    """Blob holding one conv / bn / block, for the single-layer entry points."""
    o = _Blob()
    k = layer["kind"]
    if k == "conv":
        _b_conv(o, layer)
    elif k == "bn":
        _b_bn(o, layer, act)
    else:
        _b_blocks(o, [layer])
    return o.finish()


# ----------------------------------------------------------------------------------------------
# Random-weight generator: conv/matmul N(0, 1/fan_in); BN scale U(0.5,1.5), bias N(0,0.1),
# written as mean 0 / variance 1-eps with eps 1e-20 as the exporter does
# (python/export_model_pytorch.py:188-239); matbias N(0,0.1); transformer weights N(0,0.02).


class _Gen:
    def __init__(self, seed: int, std_override=None):
        self.rng = np.random.default_rng(seed)
        self.std_override = std_override
        self.n = 0

    def name(self, base):
        self.n += 1
        return f"{base}{self.n}"

    def conv(self, k, ic, oc, base="conv"):
        std = self.std_override if self.std_override is not None else (1.0 / (k * k * ic)) ** 0.5
        w = (self.rng.standard_normal((oc, ic, k, k)) * std).astype(np.float32)
        return dict(kind="conv", name=self.name(base), kY=k, kX=k, inC=ic, outC=oc, dilY=1, dilX=1, w=w)

    def matmul(self, ic, oc, base="matmul"):
        std = self.std_override if self.std_override is not None else (1.0 / ic) ** 0.5
        return dict(kind="matmul", name=self.name(base), inC=ic, outC=oc, w=(self.rng.standard_normal((ic, oc)) * std).astype(np.float32))

    def matbias(self, c, base="bias"):
        return dict(kind="matbias", name=self.name(base), C=c, w=(self.rng.standard_normal(c) * 0.1).astype(np.float32))

    def bn(self, c, base="norm"):
        eps = np.float32(1e-20)
        return dict(kind="bn", name=self.name(base), C=c, eps=eps, hasScale=1, hasBias=1,
                    mean=np.zeros(c, np.float32), var=np.full(c, np.float32(1.0) - eps, np.float32),
                    scale=self.rng.uniform(0.5, 1.5, c).astype(np.float32), bias=(self.rng.standard_normal(c) * 0.1).astype(np.float32))

    def act(self, a, base="act"):
        return dict(kind="act", name=self.name(base), act=a)

    def trms(self, c):
        return dict(kind="trmsnorm", name=self.name("ln"), C=c, eps=np.float32(1e-6), w=np.ones(c, np.float32))


def _gen_ordinary(g: _Gen, c, mid, act):
    return dict(kind="ordinary_block", name=g.name("rblock"), preBN=g.bn(c), preAct=g.act(act), conv1=g.conv(3, c, mid),
                midBN=g.bn(mid), midAct=g.act(act), conv2=g.conv(3, mid, c))


def _gen_gpool(g: _Gen, c, regular, gpool, act):
    return dict(kind="gpool_block", name=g.name("gblock"), preBN=g.bn(c), preAct=g.act(act), regularConv=g.conv(3, c, regular),
                gpoolConv=g.conv(3, c, gpool), gpoolBN=g.bn(gpool), gpoolAct=g.act(act), gpoolToBias=g.matmul(3 * gpool, regular),
                midBN=g.bn(regular), midAct=g.act(act), finalConv=g.conv(3, regular, c))


def _gen_heads(g: _Gen, m, trunk_c, p1c, g1c, v1c, v2c, act, std_bias=True, policy_c=None):
    v = m["version"]
    # desc.cpp:1921-1934: 1 policy channel up to v11, 2 for v12-v15, 4 for v16 (q-value channels), v17 states its own
    pc = 4 if v == 16 else (2 if v >= 12 else 1)
    if policy_c is not None:
        if v < 17 and policy_c != pc:
            raise ValueError("only model version 17 chooses its number of policy channels")
        pc = policy_c
    p = dict(name="policyhead", policyC=pc, p1Conv=g.conv(1, trunk_c, p1c), g1Conv=g.conv(1, trunk_c, g1c), g1BN=g.bn(g1c), g1Act=g.act(act),
             gpoolToBias=g.matmul(3 * g1c, p1c), p1BN=g.bn(p1c), p1Act=g.act(act), p2Conv=g.conv(1, p1c, pc))
    if v >= 15:
        p["passMul"] = g.matmul(3 * g1c, p1c); p["passBias"] = g.matbias(p1c); p["passAct"] = g.act(act); p["passMul2"] = g.matmul(p1c, pc)
    else:
        p["passMul"] = g.matmul(3 * g1c, pc)
    sv = 6 if v >= 9 else (4 if v >= 8 else (2 if v >= 4 else 1))
    h = dict(name="valuehead", v1Conv=g.conv(1, trunk_c, v1c), v1BN=g.bn(v1c), v1Act=g.act(act), v2Mul=g.matmul(3 * v1c, v2c),
             v2Bias=g.matbias(v2c), v2Act=g.act(act), v3Mul=g.matmul(v2c, 3), v3Bias=g.matbias(3), sv3Mul=g.matmul(v2c, sv),
             sv3Bias=g.matbias(sv), ownConv=g.conv(1, v1c, 1))
    m["policyHead"], m["valueHead"] = p, h


_POST = [20.0, 20.0, 20.0, 20.0, 40.0, 0.25, 150.0]  # tdScore, scoreMean, scoreStdev, lead, varTime, stValueErr, stScoreErr


def make_convnet(name, seed, version, trunk_c, blocks, heads, act, mid_c=None, regular_c=None, gpool_c=None, policy_c=None):
    """blocks: list of 'plain' / 'gpool' for a plain residual net, or ('nbt', [inner kinds]) entries."""
    g = _Gen(seed)
    sp, gl = num_features(version)
    m: Dict[str, Any] = dict(name=name, version=version, numInputChannels=sp, numInputGlobalChannels=gl,
                             postProcess=_POST if version >= 13 else None, metaEncoderVersion=0)
    mid_c = mid_c or trunk_c
    t: Dict[str, Any] = dict(name="trunk", numBlocks=len(blocks), trunkC=trunk_c, midC=mid_c, regularC=regular_c, dilatedC=regular_c,
                             gpoolC=gpool_c, normKind=0)
    t["initialConv"] = g.conv(3, sp, trunk_c)
    t["initialMatMul"] = g.matmul(gl, trunk_c)
    out = []
    for b in blocks:
        if b == "plain":
            out.append(_gen_ordinary(g, trunk_c, mid_c, act))
        elif b == "gpool":
            out.append(_gen_gpool(g, trunk_c, regular_c, gpool_c, act))
        else:
            kind, inner = b
            assert kind == "nbt"
            nb = dict(kind="nested_bottleneck_block", name=g.name("nbtblock"), preBN=g.bn(trunk_c), preAct=g.act(act), preConv=g.conv(1, trunk_c, mid_c))
            nb["blocks"] = [(_gen_ordinary(g, mid_c, mid_c, act) if ik == "plain" else _gen_gpool(g, mid_c, regular_c, gpool_c, act)) for ik in inner]
            nb["postBN"] = g.bn(mid_c); nb["postAct"] = g.act(act); nb["postConv"] = g.conv(1, mid_c, trunk_c)
            out.append(nb)
    t["blocks"] = out
    t["tipBN"] = g.bn(trunk_c)
    t["tipAct"] = g.act(act)
    m["trunk"] = t
    _gen_heads(g, m, trunk_c, *heads, act, policy_c=policy_c)
    return m


def make_b6c96(seed=1000, gpool_blocks=(2,)):
    """The fp32 benchmark configuration: 6 plain residual blocks of two 3x3 convs, 96 channels, gpool in the listed block(s)."""
    blocks = ["gpool" if i in gpool_blocks else "plain" for i in range(6)]
    return make_convnet("b6c96-random", seed, 15, 96, blocks, (32, 32, 32, 64), ACT_RELU, mid_c=96, regular_c=64, gpool_c=32)


def make_nbt(name, seed, num_blocks, trunk_c, mid_c, gpool_c, heads, gpool_every=3):
    """Nested-bottleneck nets (python/katago/train/modelconfigs.py:945-981, 1349-1395): every block has two inner
    blocks; in every `gpool_every`-th block except the last one the first inner block is a pooling block."""
    blocks = []
    for i in range(num_blocks):
        first = "gpool" if (i % gpool_every) == gpool_every - 1 and i != num_blocks - 1 else "plain"
        blocks.append(("nbt", [first, "plain"]))
    return make_convnet(name, seed, 15, trunk_c, blocks, heads, ACT_MISH, mid_c=mid_c, regular_c=mid_c - gpool_c, gpool_c=gpool_c)


def add_meta_encoder(m: Dict[str, Any], seed=1500, hidden=(64, 48)) -> Dict[str, Any]:
    """Adds an SGF metadata encoder (human-SL nets; desc.cpp:1476-1522, version 1 = 192 input channels) with random
    weights to a model tree of version >= 15: 192 -> hidden[0] -> hidden[1] -> trunk channels."""
    if m["version"] < 15:
        raise ValueError("the metadata encoder needs model version >= 15")
    g = _Gen(seed)
    act = m["trunk"]["tipAct"]["act"]
    c = m["trunk"]["trunkC"]
    m["metaEncoderVersion"] = 1
    m["trunk"]["metaEncoder"] = dict(
        name="sgfmeta", numInputMetaChannels=192, mul1=g.matmul(192, hidden[0]), bias1=g.matbias(hidden[0]), act1=g.act(act),
        mul2=g.matmul(hidden[0], hidden[1]), bias2=g.matbias(hidden[1]), act2=g.act(act), mul3=g.matmul(hidden[1], c))
    return m


def random_meta_rows(n, seed=2500, channels=192):
    """Synthetic SGF metadata rows: a sparse 0/1 pattern plus a few fractional fields, as sgfmetadata.cpp fills them."""
    rng = np.random.default_rng(seed)
    rows = (rng.random((n, channels)) < 0.15).astype(np.float32)
    rows[:, -8:] = rng.random((n, 8)).astype(np.float32)
    return rows


def make_b18c384nbt(seed=1001, num_blocks=18):
    return make_nbt("b18c384nbt-random", seed, num_blocks, 384, 192, 64, (48, 48, 96, 128))


def make_b28c512nbt(seed=1002, num_blocks=28):
    return make_nbt("b28c512nbt-random", seed, num_blocks, 512, 256, 64, (64, 64, 128, 144))


def make_transformer(seed=1003, layers=12, d=384, heads=6, head_dim=64, ffn=1024, rope="learnable", rel_bias=False):
    """The transformer benchmark configuration: conv stem to d, `layers` pre-norm (attention, SwiGLU FFN) pairs, standard heads.
    Weights N(0, 0.02).  The positional scheme is RoPE, the one the reference's file format can express; rel_bias adds
    a learned per-head relative-position bias table [heads][37][37] ~ N(0, 0.2) to every attention block, which only
    the blob (to_blob) can carry."""
    g = _Gen(seed, std_override=0.02)
    v = 17
    sp, gl = num_features(v)
    m: Dict[str, Any] = dict(name="tf12d384-random", version=v, numInputChannels=sp, numInputGlobalChannels=gl, postProcess=_POST, metaEncoderVersion=0)
    t: Dict[str, Any] = dict(name="trunk", numBlocks=2 * layers, trunkC=d, midC=d, regularC=d, dilatedC=d, gpoolC=d, normKind=1)
    t["initialConv"] = g.conv(3, sp, d)
    t["initialMatMul"] = g.matmul(gl, d)
    blocks = []
    for _ in range(layers):
        a = dict(kind="transformer_attention_block", name=g.name("attn"), heads=heads, kvHeads=heads, qDim=head_dim, vDim=head_dim,
                 useRope=0 if rope == "none" else 1, learnableRope=1 if rope == "learnable" else 0, preLN=g.trms(d),
                 q=g.matmul(d, heads * head_dim), k=g.matmul(d, heads * head_dim), v=g.matmul(d, heads * head_dim), out=g.matmul(heads * head_dim, d))
        if rope == "learnable":
            a["ropeFreqs"] = g.rng.uniform(-1.0, 1.0, heads * (head_dim // 2) * 2).astype(np.float32)
        elif rope == "fixed":
            a["ropeTheta"] = np.float32(100.0)
        if rel_bias:
            a["relBias"] = (g.rng.standard_normal((heads, 37, 37)) * 0.2).astype(np.float32)
        blocks.append(a)
        blocks.append(dict(kind="transformer_ffn_block", name=g.name("ffn"), C=d, ffnC=ffn, swiglu=1, preLN=g.trms(d),
                           linear1=g.matmul(d, ffn), gate=g.matmul(d, ffn), linear2=g.matmul(ffn, d)))
    t["blocks"] = blocks
    t["tipRMSNorm"] = dict(kind="rmsnorm", name="trunk_tip", C=d, eps=np.float32(1e-6), spatial=0, gamma=np.ones(d, np.float32), beta=np.zeros(d, np.float32))
    t["tipAct"] = g.act(ACT_SILU)
    m["trunk"] = t
    _gen_heads(g, m, d, 48, 48, 96, 128, ACT_SILU)
    return m


def make_transformer_relbias(seed=1004, layers=12):
    """The transformer benchmark configuration as worded: 12 pre-norm layers of 6 heads x 64 with a learned per-head relative-position bias
    (no RoPE), SwiGLU 1024.  Only the blob can carry the bias."""
    return make_transformer(seed=seed, layers=layers, rope="none", rel_bias=True)


# ----------------------------------------------------------------------------------------------
# Synthetic positions (stand-ins for real game positions): per point empty/black/white with
# p = 0.6/0.2/0.2, plane 0 = on-board mask, planes 3.. Bernoulli(0.1) on board, global[5] = komi/20.


def random_positions(n, seed=2000, nn_len=19, board_sizes=None, num_spatial=22, num_global=19):
    """Returns (spatial [n,nn_len,nn_len,C] NHWC fp32, global [n,G] fp32).  board_sizes: per-row board edge
    (boards smaller than nn_len sit in the top-left corner, zero elsewhere)."""
    rng = np.random.default_rng(seed)
    spatial = np.zeros((n, nn_len, nn_len, num_spatial), np.float32)
    glob = np.zeros((n, num_global), np.float32)
    for i in range(n):
        bs = nn_len if board_sizes is None else int(board_sizes[i])
        stones = rng.choice(3, size=(bs, bs), p=[0.6, 0.2, 0.2])
        spatial[i, :bs, :bs, 0] = 1.0
        spatial[i, :bs, :bs, 1] = stones == 1
        spatial[i, :bs, :bs, 2] = stones == 2
        spatial[i, :bs, :bs, 3:] = rng.random((bs, bs, num_spatial - 3)) < 0.1
        glob[i] = (rng.random(num_global) < 0.5).astype(np.float32)
        if num_global > 5:
            glob[i, 5] = rng.uniform(-10.0, 10.0) / 20.0
    return spatial, glob
