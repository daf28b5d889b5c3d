"""The checkpoint reader (csrc/checkpoint.cu, q27b200/checkpoint.py): the safetensors header, the two namings of an
NVFP4 projection (engine/src/weights.cc:125-141, weights.h:71-75) and, on a GPU, the upload into the kernels' layouts -
row order, swizzled scales, interleaved gate | up (engine/src/weights.cc:177-185,218-234) - against the oracle's
host-side relayout, and the loaded layers against the oracle's GEMM."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from q27b200.checkpoint import Checkpoint, fp4_tensors, write_safetensors
from q27b200.q27lib import lib

HAS_GPU = torch.cuda.is_available()


def random_layer(rng, out, inp):
    codes = rng.randint(0, 256, size=(out, inp // 2)).astype(np.uint8)
    sf = O.e4m3_encode((rng.rand(out, inp // 16) * 2.0 + 0.25).astype(np.float32))
    return codes, sf


def make_checkpoint(path, layers, compressed):
    tensors = {}
    for prefix, (codes, sf, w2, ins) in layers.items():
        tensors.update(fp4_tensors(prefix, codes, sf, w2, ins, compressed))
    tensors["model.norm.weight"] = ("BF16", np.arange(8, dtype=np.uint16))
    write_safetensors(path, tensors, metadata={"format": "pt"})


@pytest.mark.parametrize("compressed", [False, True])
def test_reader_understands_both_namings(tmp_path, compressed):
    rng = np.random.RandomState(3)
    layers = {"model.layers.0.self_attn.q_proj": (*random_layer(rng, 256, 128), 3.5e-5, 0.0123),
              "model.layers.0.mlp.down_proj": (*random_layer(rng, 128, 320), 1.25e-4, 0.5)}
    path = str(tmp_path / "model.safetensors")
    make_checkpoint(path, layers, compressed)
    with Checkpoint(path) as ck:
        assert len(ck) == 4 * len(layers) + 1
        assert ck.tensor_info("model.norm.weight") == ("BF16", (8,), 16)
        assert ck.tensor_info("no.such.tensor") is None and not ck.has("__metadata__")
        for prefix, (codes, sf, w2, ins) in layers.items():
            li = ck.fp4_layer(prefix)
            assert (li.out, li.inp, li.compressed_tensors) == (codes.shape[0], codes.shape[1] * 2, int(compressed))
            if compressed:  # stored as reciprocals: one rounding each way
                assert abs(li.w_scale2 / w2 - 1) < 3e-7 and abs(li.in_scale / ins - 1) < 3e-7
            else:
                assert li.w_scale2 == np.float32(w2) and li.in_scale == np.float32(ins)
            name = prefix + (".weight_packed" if compressed else ".weight")
            assert np.array_equal(ck.read(name).reshape(codes.shape), codes)
            assert np.array_equal(ck.read(prefix + ".weight_scale").reshape(sf.shape), sf)


def test_reader_takes_a_directory_of_shards(tmp_path):
    rng = np.random.RandomState(4)
    a = {"a.q_proj": (*random_layer(rng, 128, 64), 1e-4, 0.1)}
    b = {"b.k_proj": (*random_layer(rng, 128, 64), 2e-4, 0.1)}
    make_checkpoint(str(tmp_path / "model-00001-of-00002.safetensors"), a, False)
    tensors = {}
    for prefix, (codes, sf, w2, ins) in b.items():
        tensors.update(fp4_tensors(prefix, codes, sf, w2, ins, True))
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), tensors)
    (tmp_path / "model.safetensors.index.json").write_text("{}")  # ignored: every shard's header says what it holds
    with Checkpoint(str(tmp_path)) as ck:
        assert ck.fp4_layer("a.q_proj").compressed_tensors == 0 and ck.fp4_layer("b.k_proj").compressed_tensors == 1
        assert abs(ck.fp4_layer("b.k_proj").w_scale2 / 2e-4 - 1) < 3e-7


def test_reader_rejects_what_it_cannot_load(tmp_path):
    rng = np.random.RandomState(5)
    codes, sf = random_layer(rng, 128, 64)
    with pytest.raises(RuntimeError, match="does not exist"):
        Checkpoint(str(tmp_path / "missing.safetensors"))
    with pytest.raises(RuntimeError, match="no .safetensors file"):
        Checkpoint(str(tmp_path))
    # a header that points past the end of the file
    bad = str(tmp_path / "bad.safetensors")
    text = json.dumps({"w": {"dtype": "U8", "shape": [4], "data_offsets": [0, 400]}}).encode()
    with open(bad, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"\0" * 4)
    with pytest.raises(RuntimeError, match="outside the file"):
        Checkpoint(bad)
    # bytes that do not match shape x dtype
    bad2 = str(tmp_path / "bad2.safetensors")
    text = json.dumps({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    with open(bad2, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    with pytest.raises(RuntimeError, match="bytes for its shape"):
        Checkpoint(bad2)
    with open(str(tmp_path / "trunc.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(RuntimeError, match="bad header length"):
        Checkpoint(str(tmp_path / "trunc.safetensors"))
    # layers that are not NVFP4 projections
    path = str(tmp_path / "odd.safetensors")
    t = fp4_tensors("ok", codes, sf, 1e-4, 0.1)
    t.update({"noscale.weight": ("U8", codes), "wrongsf.weight": ("U8", codes), "wrongsf.weight_scale": ("F8_E4M3", sf[:, :2]),
              "fp8.weight": ("F8_E4M3", codes), "half.weight": ("U8", codes), "half.weight_scale": ("F8_E4M3", sf),
              "half.weight_scale_2": ("F32", np.ones(1, np.float32)),
              "zero.weight_packed": ("U8", codes), "zero.weight_scale": ("F8_E4M3", sf),
              "zero.weight_global_scale": ("F32", np.zeros(1, np.float32)), "zero.input_global_scale": ("F32", np.ones(1, np.float32))})
    write_safetensors(path, t)
    with Checkpoint(path) as ck:
        assert ck.fp4_layer("ok").out == 128
        for prefix, msg in (("absent", "neither .weight nor .weight_packed"), ("noscale", "weight_scale is missing"),
                            ("wrongsf", r"expected F8_E4M3 \[128\]\[4\]"), ("fp8", "expected an NVFP4 matrix"),
                            ("half", "input_scale is missing"), ("zero", "reciprocal scale of 0")):
            with pytest.raises(RuntimeError, match=msg):
                ck.fp4_layer(prefix)
        with pytest.raises(RuntimeError, match=r"bytes \[0, 99999\)"):
            from q27b200.q27lib import call

            call("q27b_ckpt_read", ck._h, b"ok.weight", 0, 99999, np.empty(8, np.uint8))


def test_library_exports_the_checkpoint_entry_points():
    for name in ("q27b_copy_glu", "q27b_ckpt_open", "q27b_ckpt_close", "q27b_ckpt_count", "q27b_ckpt_tensor", "q27b_ckpt_read",
                 "q27b_ckpt_fp4_layer", "q27b_ckpt_load_fp4"):
        assert hasattr(lib(), name)


# ------------------------------------------------------------------------------------------------------ on a GPU

def quantised(rng, out, inp, sigma=0.02):
    w = (rng.randn(out, inp) * sigma).astype(np.float32)
    codes, sf, g = O.quant_weight_rtn(w)
    return codes, sf, float(g)


@pytest.mark.gpu
@pytest.mark.parametrize("compressed", [False, True])
def test_upload_lays_the_weights_out_for_the_kernels(tmp_path, compressed):
    """Codes in row order, scales in swizzled atoms, fused projections adjacent, gate | up interleaved in blocks of 64
    rows: byte for byte what the oracle's host-side relayout of the same tensors gives. The gate | up matrix is larger
    than one staging piece would need to be to show the strided copy (64-row blocks of 2560 bytes)."""
    rng = np.random.RandomState(11)
    K, I = 5120, 1152
    layers = {"l.q_proj": (*quantised(rng, 512, K), 0.01), "l.k_proj": (*quantised(rng, 128, K), 0.01),
              "l.v_proj": (*quantised(rng, 128, K), 0.01), "l.mlp.gate_proj": (*quantised(rng, I, K), 0.02),
              "l.mlp.up_proj": (*quantised(rng, I, K), 0.02), "l.mlp.down_proj": (*quantised(rng, 640, I), 0.04)}
    path = str(tmp_path / "m.safetensors")
    make_checkpoint(path, layers, compressed)
    with Checkpoint(path) as ck:
        q = ck.load_fp4("l.q_proj")
        codes, sf, g, ins = layers["l.q_proj"]
        assert np.array_equal(q.w.cpu().numpy(), codes) and np.array_equal(q.sf.cpu().numpy(), O.swizzle_sf(sf))
        assert (q.out, q.inp, q.glu) == (512, K, False)
        f = ck.load_fp4_fused(["l.q_proj", "l.k_proj", "l.v_proj"])
        parts = [layers[n] for n in ("l.q_proj", "l.k_proj", "l.v_proj")]
        assert np.array_equal(f.w.cpu().numpy(), np.concatenate([p[0] for p in parts]))
        assert np.array_equal(f.sf.cpu().numpy(), O.swizzle_sf(np.concatenate([p[1] for p in parts])))
        assert list(f._zero) == [0, 512, 640] and f.rows() == 768
        for a, p in zip(f._alpha, parts):
            assert abs(a / (np.float32(p[3]) * np.float32(p[2])) - 1) < 1e-6
        gu, ag, au = ck.load_fp4_glu("l.mlp.gate_proj", "l.mlp.up_proj")
        gate, up = layers["l.mlp.gate_proj"], layers["l.mlp.up_proj"]
        assert np.array_equal(gu.w.cpu().numpy(), O.interleave_glu(np.concatenate([gate[0], up[0]])))
        assert np.array_equal(gu.sf.cpu().numpy(), O.swizzle_sf(O.interleave_glu(np.concatenate([gate[1], up[1]]))))
        assert gu.glu and gu.out == I and gu.rows() == 2 * I
        assert abs(ag / (0.02 * gate[2]) - 1) < 1e-6 and abs(au / (0.02 * up[2]) - 1) < 1e-6 and ag != au


@pytest.mark.gpu
def test_copy_glu_pieces_that_start_inside_a_block():
    """The interleaving copy takes any byte range of a half: a piece may start and end inside a 64-row block."""
    from q27b200.q27lib import call

    rng = np.random.RandomState(12)
    block, blocks = 64 * 48, 5
    halves = [rng.randint(0, 256, size=blocks * block).astype(np.uint8) for _ in range(2)]
    dst = torch.zeros(2 * blocks * block, dtype=torch.uint8, device="cuda")
    cuts = [0, 100, block - 1, block + 7, 3 * block, 3 * block + 1, blocks * block]
    pinned = [torch.from_numpy(h).pin_memory() for h in halves]
    for half in (0, 1):
        for a, b in zip(cuts[:-1], cuts[1:]):
            call("q27b_copy_glu", dst, a, pinned[half].data_ptr() + a, b - a, block, half, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    want = np.stack([halves[0].reshape(blocks, block), halves[1].reshape(blocks, block)], axis=1).reshape(-1)
    assert np.array_equal(dst.cpu().numpy(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [3, 200])
def test_loaded_mlp_matches_the_oracle(tmp_path, M):
    """A checkpoint's MLP (gate and up with tensor scales of their own, compressed-tensors naming) through the loaded
    layers - weight-streaming kernels at 3 tokens, the many-row kernels with the NVFP4 epilogue at 200 - against the
    oracle: down(quant(silu(a_g gate) * (a_u up)))."""
    rng = np.random.RandomState(13)
    K, I = 1024, 1152
    gate, up, down = quantised(rng, I, K, 0.03), quantised(rng, I, K, 0.05), quantised(rng, 1024, I, 0.04)
    in_h, in_d = 0.011, 0.007
    layers = {"m.gate_proj": (*gate, in_h), "m.up_proj": (*up, in_h), "m.down_proj": (*down, in_d)}
    path = str(tmp_path / "mlp.safetensors")
    make_checkpoint(path, layers, True)
    with Checkpoint(path) as ck:
        mlp = ck.load_mlp("m")
    x = (rng.randn(M, K) * 1.0).astype(np.float32)
    got = mlp(torch.from_numpy(x).cuda()).cpu().numpy()
    li_scale = lambda v: float(np.float32(1.0) / (np.float32(1.0) / np.float32(v)))  # noqa: E731  (what the file holds)
    xq = O.quant_act_nvfp4(x, li_scale(in_h)).astype(np.float64)
    g = xq @ O.dequant_nvfp4(gate[0], gate[1], li_scale(gate[2])).astype(np.float64).T
    u = xq @ O.dequant_nvfp4(up[0], up[1], li_scale(up[2])).astype(np.float64).T
    h = O.silu_mul(g.astype(np.float32), u.astype(np.float32))
    hq = O.quant_act_nvfp4(h, li_scale(in_d)).astype(np.float64)
    want = hq @ O.dequant_nvfp4(down[0], down[1], li_scale(down[2])).astype(np.float64).T
    # the intermediate is re-quantised: a value next to a rounding boundary may land on the other code in fp32, so the
    # comparison is on the whole matrix, not element by element
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 2e-3, err
