"""Host logic: model-file reader/writer, generator and blob serialiser (no GPU)."""
import os
import subprocess

import numpy as np
import pytest

from katago_b200 import modelfile as mf

REF_MODELS = os.path.join(os.environ.get("KATAGO_REFERENCE", "/root/reference"), "cpp", "tests", "models")
REF_TOOL = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "modelfile_to_blob")


def test_writer_reader_roundtrip_bit_exact():
    for model in (mf.make_b6c96(), mf.make_b18c384nbt(num_blocks=2), mf.make_transformer(layers=1, d=64, heads=2, head_dim=32, ffn=96)):
        data = mf.model_file_bytes(model)
        again = mf.parse_model_bytes(data, True)
        assert mf.to_blob(again) == mf.to_blob(model)


def test_generator_shapes_match_named_configs():
    m = mf.make_b18c384nbt()
    kinds = [b["blocks"][0]["kind"] for b in m["trunk"]["blocks"]]
    assert len(kinds) == 18 and kinds.count("gpool_block") == 5 and kinds[17] == "ordinary_block"
    assert m["trunk"]["trunkC"] == 384 and m["trunk"]["midC"] == 192 and m["trunk"]["gpoolC"] == 64
    m = mf.make_b28c512nbt()
    kinds = [b["blocks"][0]["kind"] for b in m["trunk"]["blocks"]]
    assert len(kinds) == 28 and kinds.count("gpool_block") == 9
    m = mf.make_b6c96()
    assert [b["kind"] for b in m["trunk"]["blocks"]].count("gpool_block") == 1


def test_generator_is_deterministic():
    assert mf.to_blob(mf.make_b6c96(seed=5)) == mf.to_blob(mf.make_b6c96(seed=5))
    assert mf.to_blob(mf.make_b6c96(seed=5)) != mf.to_blob(mf.make_b6c96(seed=6))


def test_reader_rejects_bad_input():
    data = mf.model_file_bytes(mf.make_b6c96())
    with pytest.raises(ValueError):
        mf.parse_model_bytes(data[: len(data) // 2], True)  # truncated
    with pytest.raises(ValueError):
        mf.parse_model_bytes(data, False)  # binary blocks read as text
    bad = bytearray(data)
    at = bad.find(b"@BIN@") + 5
    bad[at : at + 4] = np.array([np.nan], "<f4").tobytes()
    with pytest.raises(ValueError):
        mf.parse_model_bytes(bytes(bad), True)  # non-finite weight (desc.cpp:21-26)


def test_random_positions_scheme():
    sp, gl = mf.random_positions(64, seed=2000, board_sizes=[19, 13, 9, 19] * 16)
    assert sp.shape == (64, 19, 19, 22) and gl.shape == (64, 19)
    assert set(np.unique(sp)) <= {0.0, 1.0}
    assert sp[1, 13:, :, :].sum() == 0 and sp[1, :, 13:, :].sum() == 0 and sp[1, :13, :13, 0].min() == 1
    stones = sp[0, :, :, 1] + sp[0, :, :, 2]
    assert stones.max() <= 1.0 and 0.25 < stones.mean() < 0.55
    assert np.all(np.abs(gl[:, 5]) <= 0.5)


@pytest.mark.skipif(not (os.path.isdir(REF_MODELS) and os.path.exists(REF_TOOL)), reason="needs the reference checkout and oracle/_ref")
@pytest.mark.parametrize("name", [
    "g170-b6c96-s175395328-d26788732.bin.gz", "g103-b6c96-s103408384-d26419149.txt.gz",
    "b7c96h3tfrs-test5-cnorm.bin.gz", "b7c96h6kv3qk32v16tflrs-fson-bnh.bin.gz"])
def test_python_reader_agrees_with_reference_loader(name, oracle, tmp_path):
    """Blob from this package's reader vs blob from the reference's own ModelDesc loader, compared through the
    oracle (the loader rescales some channels, desc.cpp:2631, so weights differ by exactly equivalent factors)."""
    out = tmp_path / "ref.blob"
    subprocess.run([REF_TOOL, os.path.join(REF_MODELS, name), str(out)], check=True, stdout=subprocess.DEVNULL)
    blob_ref = out.read_bytes()
    blob_py = mf.to_blob(mf.load_model_file(os.path.join(REF_MODELS, name)))
    a, b = oracle.OracleModel(blob_ref), oracle.OracleModel(blob_py)
    sp, gl = mf.random_positions(2, seed=5, num_spatial=a.in_c, num_global=a.in_global_c, board_sizes=[19, 11])
    oa, ob = a.forward(sp, gl), b.forward(sp, gl)
    for k in oa:
        assert np.abs(oa[k] - ob[k]).max() <= 1e-4 * max(1.0, np.abs(oa[k]).max()), k


def _meta_model():
    return mf.add_meta_encoder(mf.make_b18c384nbt(seed=31, num_blocks=2))


def test_meta_encoder_roundtrip_and_oracle(oracle):
    """SGF metadata encoder (human-SL nets): writer -> reader round trip is bit exact, the blob carries the encoder,
    and the oracle requires metadata rows exactly for such nets."""
    m = _meta_model()
    raw = mf.model_file_bytes(m)
    m2 = mf.parse_model_bytes(raw, True)
    assert mf.to_blob(m) == mf.to_blob(m2)
    om = oracle.OracleModel(mf.to_blob(m))
    sp, gl = mf.random_positions(3, seed=5)
    meta = mf.random_meta_rows(3)
    a = om.forward(sp, gl, meta=meta)
    b = om.forward(sp, gl, meta=np.zeros_like(meta))
    assert np.abs(a["value"] - b["value"]).max() > 1e-4   # the rows reach the trunk
    with pytest.raises(Exception):
        om.forward(sp, gl)
    plain = oracle.OracleModel(mf.to_blob(mf.make_b18c384nbt(seed=31, num_blocks=2)))
    with pytest.raises(Exception):
        plain.forward(sp, gl, meta=meta)


@pytest.mark.skipif(not os.path.exists(REF_TOOL), reason="needs oracle/_ref")
def test_reference_loader_accepts_generated_meta_encoder_file(oracle, tmp_path):
    """A generated model file with a metadata encoder goes through the reference's own ModelDesc loader and the
    backend's ModelDesc -> blob conversion, and evaluates like the blob made directly from the generator's tree."""
    m = _meta_model()
    path = tmp_path / "meta.bin.gz"
    mf.save_model_file(m, str(path))
    out = tmp_path / "ref.blob"
    subprocess.run([REF_TOOL, str(path), str(out)], check=True, stdout=subprocess.DEVNULL)
    a, b = oracle.OracleModel(out.read_bytes()), oracle.OracleModel(mf.to_blob(m))
    sp, gl = mf.random_positions(2, seed=6, board_sizes=[19, 13])
    meta = mf.random_meta_rows(2, seed=7)
    oa, ob = a.forward(sp, gl, meta=meta), b.forward(sp, gl, meta=meta)
    for k in oa:
        assert np.abs(oa[k] - ob[k]).max() <= 1e-4 * max(1.0, np.abs(oa[k]).max()), k



def _relbias_model():
    return mf.make_transformer(seed=41, layers=2, d=64, heads=2, head_dim=32, ffn=96, rope="none", rel_bias=True)


def test_extension_file_roundtrip_and_checks(tmp_path):
    """A net with a learned relative-position attention bias is stored as an ordinary model file plus the extension
    file <model file>.kbext: the pair reads back to the same blob; the model file alone is the same net without the
    bias; a model without such weights writes no extension file (and removes a stale one); malformed or mismatched
    extension files are rejected."""
    m = _relbias_model()
    path = str(tmp_path / "rb.bin.gz")
    mf.save_model_file(m, path)
    assert os.path.exists(path + mf.EXT_SUFFIX)
    assert mf.to_blob(mf.load_model_file(path)) == mf.to_blob(m)
    bare = mf.parse_model_bytes(mf.model_file_bytes(m), True)
    assert all(b.get("relBias") is None for b in bare["trunk"]["blocks"])
    assert mf.to_blob(bare) != mf.to_blob(m)
    ext = mf.model_ext_bytes(m)
    # the same checks as the C++ reader (katago_b200/host/model_ext.h)
    for bad, what in [
        (ext[:-4], "past the end"), (ext[:10], "truncated"), (ext + b"\0\0\0\0", "after the last record"), (b"KBMDLEXX" + ext[8:], "not a model extension"),
        (ext[:8] + (2).to_bytes(4, "little") + ext[12:], "version"),
    ]:
        with pytest.raises(ValueError, match=what):
            mf.attach_model_ext(mf.parse_model_bytes(mf.model_file_bytes(m), True), bad)
    other = mf.parse_model_bytes(mf.model_file_bytes(m), True)
    other["name"] = "another-net"
    with pytest.raises(ValueError, match="written for model"):
        mf.attach_model_ext(other, ext)
    renamed = mf.parse_model_bytes(mf.model_file_bytes(m), True)
    renamed["trunk"]["blocks"][0]["name"] = "elsewhere"
    with pytest.raises(ValueError, match="does not have"):
        mf.attach_model_ext(renamed, ext)
    plain = mf.make_b6c96()
    assert mf.model_ext_bytes(plain) is None
    mf.save_model_file(plain, path)
    assert not os.path.exists(path + mf.EXT_SUFFIX)


@pytest.mark.skipif(not os.path.exists(REF_TOOL), reason="needs oracle/_ref")
def test_reference_loader_plus_extension_file_gives_the_generators_net(oracle, tmp_path):
    """The route a backend takes: the reference's own loader parses the model file, the extension file's records are
    attached by block name while the ModelDesc is flattened (katago_b200/host/modeldesc_blob.h), and the result
    evaluates like the blob made directly from the generator's tree; without the extension file the bias is absent."""
    m = _relbias_model()
    path = tmp_path / "rb.bin.gz"
    mf.save_model_file(m, str(path))
    out = tmp_path / "ref.blob"
    subprocess.run([REF_TOOL, str(path), str(out)], check=True, stdout=subprocess.DEVNULL)
    with_ext = out.read_bytes()
    assert len(with_ext) == len(mf.to_blob(m))
    a, b = oracle.OracleModel(with_ext), oracle.OracleModel(mf.to_blob(m))
    sp, gl = mf.random_positions(2, seed=6, board_sizes=[19, 13])
    oa, ob = a.forward(sp, gl), b.forward(sp, gl)
    for k in oa:
        assert np.abs(oa[k] - ob[k]).max() <= 1e-5 * max(1.0, np.abs(oa[k]).max()), k
    os.remove(str(path) + mf.EXT_SUFFIX)
    subprocess.run([REF_TOOL, str(path), str(out)], check=True, stdout=subprocess.DEVNULL)
    bias_words = sum(b["relBias"].size + 3 + 3 for b in m["trunk"]["blocks"] if b.get("relBias") is not None)
    assert len(out.read_bytes()) == len(with_ext) - 4 * bias_words
    oc = oracle.OracleModel(out.read_bytes()).forward(sp, gl)
    assert np.abs(oc["policy"] - ob["policy"]).max() > 1e-5
    # an extension file that names a block the model does not have is refused by the C++ reader too
    renamed = _relbias_model()
    renamed["trunk"]["blocks"][0]["name"] = "elsewhere"
    with open(str(path) + mf.EXT_SUFFIX, "wb") as f:
        f.write(mf.model_ext_bytes(renamed))
    r = subprocess.run([REF_TOOL, str(path), str(out)], capture_output=True, text=True)
    assert r.returncode != 0 and "does not have" in r.stderr
