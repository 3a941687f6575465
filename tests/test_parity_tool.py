"""The `parity spconv` tool: reader / writer of the reference's dump container, the compare line, and (GPU) a whole run on
a dump written in the format of tools/ref_spconv.py of trellis2-cuda."""
import io

import numpy as np
import pytest
import torch

from trellis2_cuda_b200 import parity, scenes


def test_safetensors_container_matches_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    g = torch.Generator().manual_seed(0)
    tensors = {"conv0/in": torch.randn(5, 8, generator=g).half(), "conv0/out": torch.randn(5, 4, generator=g).bfloat16(),
               "conv0/coords": torch.randint(0, 100, (5, 4), generator=g, dtype=torch.int32),
               "conv0/name": torch.tensor(list(b"blocks.0.0.conv"), dtype=torch.uint8), "w": torch.randn(3, 3, generator=g)}
    mine, theirs = str(tmp_path / "mine.safetensors"), str(tmp_path / "theirs.safetensors")
    parity.write_safetensors(mine, tensors)
    st.save_file(tensors, theirs)
    for a, b in ((st.load_file(mine), tensors), (parity.read_safetensors(theirs), tensors), (parity.read_safetensors(mine), tensors)):
        assert set(a) == set(b)
        for k in b:
            assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape and torch.equal(a[k], b[k]), k
    assert bytes(parity.read_safetensors(theirs)["conv0/name"].tolist()).decode() == "blocks.0.0.conv"


def test_cmp_line_counts_like_the_reference_harness():
    a = torch.tensor([1.0, 2.0, 3.0, -4.0]).half()
    b = torch.tensor([1.0, 2.5, 3.0, -4.0]).half()
    text, nbad, mx, mr = parity.cmp_line("conv0/x", a, b)
    assert nbad == 1 and abs(mx - 0.5) < 1e-6 and abs(mr - 0.5 / 10.5) < 1e-6
    assert "4 elems" in text and "mismatch          1" in text and "maxabs 0.5" in text and "(ref max 4)" in text
    text, nbad, _, _ = parity.cmp_line("conv0/x", a, b.float())
    assert "[dtype differs]" in text and nbad == 1
    assert "MISMATCH" in parity.cmp_line("conv0/x", a, b[:3])[0]


@pytest.mark.gpu
def test_parity_spconv_on_a_dump_in_the_reference_format(tmp_path):
    """Two convs dumped the way tools/ref_spconv.py dumps them - inputs, coordinates, module name and the output of the
    reference's own CUDA kernel (oracle/_ref) where that library was built, else of the CPU oracle - plus a checkpoint with
    [Co,3,3,3,Ci] weights: the tool must report both within tolerance, and --strict must count the differing elements."""
    import oracle
    from oracle import ref
    rng = np.random.default_rng(3)
    dump, ckpt = {}, {}
    for j, (n, res, Ci, Co, name) in enumerate(((1500, 13, 64, 64, "blocks.3.0.conv"), (900, 11, 128, 256, "blocks.2.1.conv1"))):
        cells = rng.choice(res ** 3, size=n, replace=False)
        c = np.stack([np.zeros(n, np.int64), cells // (res * res), (cells // res) % res, cells % res], 1).astype(np.int32)
        x = rng.standard_normal((n, Ci)).astype(np.float16)
        w = scenes.kaiming_uniform_weight(Co, Ci, 7 + j).astype(np.float16)
        b = (0.1 * rng.standard_normal(Co)).astype(np.float16)
        if ref.available(False):
            y = ref.subm_conv(c, x, w, b)[0]
        else:
            y = oracle.conv_block(x.astype(np.float32), w.astype(np.float32), b.astype(np.float32), oracle.build_neighbors(c)[0], "f16").astype(np.float16)
        dump[f"conv{j}/in"], dump[f"conv{j}/out"], dump[f"conv{j}/coords"] = torch.from_numpy(x), torch.from_numpy(y), torch.from_numpy(c)
        dump[f"conv{j}/name"] = torch.tensor(list(name.encode()), dtype=torch.uint8)
        ckpt[name + ".weight"] = torch.from_numpy(w).reshape(Co, 3, 3, 3, Ci)
        ckpt[name + ".bias"] = torch.from_numpy(b)
    parity.write_safetensors(str(tmp_path / "spconv.safetensors"), dump)
    parity.write_safetensors(str(tmp_path / "dec.safetensors"), ckpt)
    out = io.StringIO()
    assert parity.parity_spconv(str(tmp_path), str(tmp_path / "dec.safetensors"), out=out) == 0
    text = out.getvalue()
    assert "conv0/blocks.3.0.conv" in text and "conv1/blocks.2.1.conv1" in text and "PARITY OK" in text
    assert "N=1500 Ci=64 Co=64 B1=128 BK=64 S=1" in text and text.count("within tolerance") == 2
    strict = io.StringIO()
    fails = parity.parity_spconv(str(tmp_path), str(tmp_path / "dec.safetensors"), strict=True, out=strict)
    assert ("PARITY OK" in strict.getvalue()) == (fails == 0)
    # command line entry
    assert parity.main(["spconv", "--ref", str(tmp_path / "spconv.safetensors"), "--ckpt", str(tmp_path / "dec.safetensors")]) == 0
