"""The packed-weight file format (python/spark_kernels/packfile.py): round trip, alignment, checksums on the
CPU; on the GPU a stored projection gives the stored object's bits without re-quantizing."""

import os

import pytest
import torch


def _pf():
    import importlib.util
    import sys

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(here, "5090-blackwell-kernels_b200", "python", "spark_kernels", "packfile.py")
    spec = importlib.util.spec_from_file_location("spk_packfile_standalone", path)  # no CUDA library needed for the container
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_round_trip_alignment_and_checksums(tmp_path):
    pf = _pf()
    g = torch.Generator().manual_seed(0)
    tensors = {"packed": torch.randint(-2 ** 31, 2 ** 31 - 1, (8, 256), dtype=torch.int32, generator=g),
               "scales": torch.randn(1, 128, generator=g).to(torch.bfloat16), "zeros": None,
               "bytes": torch.randint(0, 255, (3, 5), dtype=torch.uint8, generator=g), "sw": torch.randn(1, generator=g),
               "scalar": torch.tensor(7.8e-5), "none": torch.zeros(0, dtype=torch.uint8)}
    path = str(tmp_path / "w.spkw")
    pf.save_tensors(path, "Int4Linear", tensors, {"note": "x"})
    kind, meta, got = pf.load_tensors(path)
    assert kind == "Int4Linear" and meta == {"note": "x"} and set(got) == {"packed", "scales", "bytes", "sw", "scalar", "none"}
    for k, t in got.items():
        assert t.dtype == tensors[k].dtype and t.shape == tensors[k].shape
        assert torch.equal(t.reshape(-1).view(torch.uint8), tensors[k].reshape(-1).view(torch.uint8))
    raw = open(path, "rb").read()
    assert raw[:8] == pf.MAGIC
    import json, struct
    header = json.loads(raw[16:16 + struct.unpack("<Q", raw[8:16])[0]])
    assert all(e["offset"] % pf.ALIGN == 0 for e in header["tensors"].values())
    # one flipped payload bit is caught; so are a bad magic and a cut file
    off = header["tensors"]["packed"]["offset"]
    bad = bytearray(raw)
    bad[off + 3] ^= 1
    open(path, "wb").write(bytes(bad))
    with pytest.raises(ValueError, match="checksum"):
        pf.load_tensors(path)
    open(path, "wb").write(b"NOTSPKW0" + raw[8:])
    with pytest.raises(ValueError, match="magic"):
        pf.load_tensors(path)
    open(path, "wb").write(raw[:off + 10])
    with pytest.raises(ValueError, match="truncated"):
        pf.load_tensors(path)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["int4", "int4-asym", "fp8-tok", "mxfp8", "nvfp4", "mxfp4"])
def test_stored_projection_gives_the_same_bits(sk, tmp_path, fmt):
    from spark_kernels import packfile

    w = (torch.randn(512, 256, device="cuda") / 22).to(torch.bfloat16)
    a = torch.randn(9, 512, device="cuda").to(torch.bfloat16)
    lin = sk.make_linear(w, fmt)
    path = str(tmp_path / f"{fmt}.spkw")
    packfile.save_linear(path, lin)
    again = packfile.load_linear(path)
    assert type(again) is type(lin) and torch.equal(again(a), lin(a))


@pytest.mark.gpu
def test_stored_gate_up_weight(sk, tmp_path):
    from spark_kernels import packfile

    w = (torch.randn(512, 256, device="cuda") / 22).to(torch.bfloat16)
    a = torch.randn(5, 512, device="cuda").to(torch.bfloat16)
    ww = sk.W4GateUpWeight.quantize(w)
    path = str(tmp_path / "gu.spkw")
    packfile.save_linear(path, ww)
    again = packfile.load_linear(path)
    assert torch.equal(sk.w4gemm_swiglu(a, again), sk.w4gemm_swiglu(a, ww))
