"""CPU: tile-config cache semantics of gemlite/core.py:838-906 and get_closest_m (utils.py:182-220)."""
import json
import os


def ref_closest_m(M, max_m=4096):
    vals = set()
    i = 0
    while 2 ** i <= max_m:
        v, nxt = 2 ** i, 2 ** (i + 1)
        vals.add(v)
        if v >= 32 and nxt <= max_m:
            vals.add((v + nxt) // 2)
            vals.add((v + nxt) // 4)
        i += 1
    if M > max_m:
        return max_m
    return min(x for x in vals if x >= M)


def test_closest_m_table(lib):
    for M in list(range(0, 300)) + [383, 384, 385, 1000, 1536, 1537, 3072, 3073, 4096, 4097, 100000]:
        assert lib.gl_get_closest_m(M) == ref_closest_m(M), M


def test_load_merge_save_reset(lib, tmp_path):
    from gemlite_b200 import GemLiteLinear
    GemLiteLinear.reset_config()
    f1 = tmp_path / "a.json"
    f1.write_text(json.dumps({"GEMM": {"(64, 8, 8, 128, 8, 104)": {"BLOCK_SIZE_M": 64, "num_warps": 4}},
                              "GEMV": {"(1, 8, 8, 128, 8, 104)": {"BLOCK_SIZE_N": 256}}}))
    assert GemLiteLinear.load_config(str(f1)) is True
    assert lib.gl_cfg_size(b"GEMM") == 1 and lib.gl_cfg_size(None) == 2
    f2 = tmp_path / "b.json"
    f2.write_text(json.dumps({"GEMM": {"(64, 8, 8, 128, 8, 104)": {"BLOCK_SIZE_M": 128},
                                       "(128, 8, 8, 128, 8, 104)": {"BLOCK_SIZE_M": 16}}}))
    assert GemLiteLinear.load_config(str(f2)) is True          # merge: same signature is replaced
    assert json.loads(lib.gl_cfg_get(b"GEMM", b"(64, 8, 8, 128, 8, 104)")) == {"BLOCK_SIZE_M": 128}
    assert lib.gl_cfg_size(None) == 3
    out = tmp_path / "c.json"
    out.write_text(json.dumps({"GEMM": {"(1, 1, 1, 1, 1, 1)": {"x": [1, 2, {"y": None}]}}}))
    GemLiteLinear.cache_config(str(out))                        # merges into what the file already holds
    saved = json.loads(out.read_text())
    assert set(saved) == {"GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"}
    assert saved["GEMM"]["(1, 1, 1, 1, 1, 1)"] == {"x": [1, 2, {"y": None}]}
    assert saved["GEMM"]["(128, 8, 8, 128, 8, 104)"] == {"BLOCK_SIZE_M": 16}
    assert GemLiteLinear.load_config(str(f1), overwrite=True) is True
    assert lib.gl_cfg_size(None) == 2
    GemLiteLinear.reset_config()
    assert lib.gl_cfg_size(None) == 0


def test_load_failures_return_false(lib, tmp_path, caplog):
    from gemlite_b200 import GemLiteLinear
    assert GemLiteLinear.load_config(None) is False
    assert GemLiteLinear.load_config(str(tmp_path / "missing.json"), print_error=False) is False
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    assert GemLiteLinear.load_config(str(bad)) is False
    assert lib.gl_cfg_set(b"GEMM", b"sig", b"{broken") != 0
