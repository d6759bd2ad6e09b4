"""Run-time proof of the drop-in route: the reference's OWN callers of the three kernel launchers,
compiled unchanged (oracle/Makefile, target `callers`), run with libpaged_attention.so in place of the
reference's flashattention.cu, rope.cu and layout.cu.

  * src/kernels/flashattention/stress_test_flashattention.cu (calls launch_flash_attention at
    :527 and :567 for sequence lengths 32 ... 2048, bf16, 32/8 heads, d = 64): must run to the end.
  * src/runtime/attention.cu — Attention::forward, which calls all three launchers (:226, :334,
    :354) — driven by oracle/attention_driver.cu through a 37-token prompt and two decode steps;
    the same driver linked against the reference's own kernels gives the expected bytes."""
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _have(name):
    return os.path.exists(os.path.join(REF_DIR, name))


@pytest.mark.skipif(not _have("stress_test_flashattention_shim"), reason="the reference's callers were not built")
def test_reference_stress_test_runs_on_the_shims(cuda):
    r = subprocess.run([os.path.join(REF_DIR, "stress_test_flashattention_shim")], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "2048" in r.stdout and "TFLOP" in r.stdout.upper()


@pytest.mark.skipif(not (_have("attention_forward_shim") and _have("attention_forward_ref")),
                    reason="the reference's callers were not built")
def test_reference_attention_forward_on_the_shims_equals_reference_kernels(cuda, tmp_path):
    outs = {}
    for name in ("attention_forward_shim", "attention_forward_ref"):
        path = tmp_path / (name + ".bin")
        r = subprocess.run([os.path.join(REF_DIR, name), str(path)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, name + ": " + r.stdout[-2000:] + r.stderr[-2000:]
        outs[name] = np.fromfile(path, dtype=np.uint16)
    got, want = outs["attention_forward_shim"], outs["attention_forward_ref"]
    prompt, n_out = 37, (37 + 2) * 2048
    assert got.size == want.size == n_out + 2 * 8 * (prompt + 2) * 64
    # caches: RoPE'd K and V as appended by the reference's own copy loop — bit for bit
    assert np.array_equal(got[n_out:], want[n_out:]), "caches differ"
    # outputs: the attention kernels differ in rounding, the output projection is the reference's GEMM
    g = orc.bf16_to_f32(got[:n_out]).astype(np.float64).reshape(-1, 2048)
    w = orc.bf16_to_f32(want[:n_out]).astype(np.float64).reshape(-1, 2048)
    err = np.abs(g - w).max(axis=1)
    scale = np.abs(w).max(axis=1)
    assert np.all(scale > 0) and np.all(err <= 2.0 ** -6 * scale), (err / scale).max()


@pytest.mark.skipif(not _have("attention_forward_ref"), reason="the reference's callers were not built")
def test_drop_in_attention_class_equals_reference_attention(cuda, tmp_path):
    """include/attention.hpp: the runtime::Attention-shaped class over the paged library (RMSNorm,
    projections, RoPE + append, attention and output projection all from this library), driven by
    the same program, against the reference's own Attention with its own kernels throughout."""
    root = os.path.dirname(REF_DIR.rstrip("/"))
    repo = os.path.dirname(root)
    exe = tmp_path / "attention_class_shim"
    r = subprocess.run(["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
                        "-DPA_SHIM_CLASS", "-I", os.path.join(repo, "include"), "-o", str(exe),
                        os.path.join(root, "attention_driver.cu"),
                        "-L", os.path.join(repo, "llama_transformer_runtime_b200"), "-lpaged_attention",
                        "-Xlinker", "-rpath", "-Xlinker", os.path.join(repo, "llama_transformer_runtime_b200")],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    outs = {}
    for name, cmd in (("shim", str(exe)), ("ref", os.path.join(REF_DIR, "attention_forward_ref"))):
        path = tmp_path / (name + ".bin")
        r = subprocess.run([cmd, str(path)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, name + ": " + r.stdout[-2000:] + r.stderr[-2000:]
        outs[name] = np.fromfile(path, dtype=np.uint16)
    got, want = outs["shim"], outs["ref"]
    prompt, n_out = 37, (37 + 2) * 2048
    assert got.size == want.size
    # caches: K passes through this library's projection GEMM (one ulp apart from the reference's
    # in places) and RoPE; V through the GEMM only
    gc = orc.bf16_to_f32(got[n_out:]).astype(np.float64)
    wc = orc.bf16_to_f32(want[n_out:]).astype(np.float64)
    assert np.all(np.abs(gc - wc) <= 2.0 ** -6 * np.maximum(np.abs(wc), 1.0)), np.abs(gc - wc).max()
    assert float((got[n_out:] == want[n_out:]).mean()) > 0.8
    g = orc.bf16_to_f32(got[:n_out]).astype(np.float64).reshape(-1, 2048)
    w = orc.bf16_to_f32(want[:n_out]).astype(np.float64).reshape(-1, 2048)
    err = np.abs(g - w).max(axis=1)
    scale = np.abs(w).max(axis=1)
    assert np.all(err <= 2.0 ** -5 * scale), (err / scale).max()


@pytest.mark.skipif(not _have("ffn_forward_ref"), reason="the reference's callers were not built")
def test_drop_in_feed_forward_class_equals_reference_feed_forward(cuda, tmp_path):
    """include/ffn.hpp: the runtime::FeedForward-shaped class over this library (1 and 3 rows through the
    weight-streaming kernels, 40 rows through the tensor-core GEMMs), driven by the same program as the
    reference's own FeedForward with its own kernels (src/runtime/ffn.cu)."""
    root = os.path.dirname(REF_DIR.rstrip("/"))
    repo = os.path.dirname(root)
    exe = tmp_path / "ffn_class_shim"
    r = subprocess.run(["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
                        "-DPA_SHIM_CLASS", "-I", os.path.join(repo, "include"), "-o", str(exe),
                        os.path.join(root, "ffn_driver.cu"),
                        "-L", os.path.join(repo, "llama_transformer_runtime_b200"), "-lpaged_attention",
                        "-Xlinker", "-rpath", "-Xlinker", os.path.join(repo, "llama_transformer_runtime_b200")],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    outs = {}
    for name, cmd in (("shim", str(exe)), ("ref", os.path.join(REF_DIR, "ffn_forward_ref"))):
        path = tmp_path / (name + ".bin")
        r = subprocess.run([cmd, str(path)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, name + ": " + r.stdout[-2000:] + r.stderr[-2000:]
        outs[name] = np.fromfile(path, dtype=np.uint16)
    got, want = outs["shim"], outs["ref"]
    assert got.size == want.size == (1 + 3 + 40) * 2048
    g = orc.bf16_to_f32(got).astype(np.float64).reshape(-1, 2048)
    w = orc.bf16_to_f32(want).astype(np.float64).reshape(-1, 2048)
    err = np.abs(g - w).max(axis=1)
    scale = np.abs(w).max(axis=1)
    assert np.all(scale > 0) and np.all(err <= 2.0 ** -6 * scale), (err / scale).max()


@pytest.mark.skipif(not _have("token_forward_ref"), reason="the reference's callers were not built")
def test_whole_model_equals_the_reference_transformer(cuda, tmp_path):
    """The reference's own runtime::Transformer (16 blocks of its Attention and FeedForward classes,
    compiled unchanged, with its kernels) inside the calls of LlamaRuntime::forward_prefill and
    decode_forward, against this library twice: the same calls on the drop-in classes and entry points
    (include/transformer.hpp, pa_embedding, pa_lm_head, pa_argmax: -DPA_SHIM_CLASS), and every token as
    one pa_decode_token step (-DPA_SHIM).  One seeded Llama-3.2-1B-shaped model, an empty cache, a
    21-token prompt, twelve steps on the same fed ids (oracle/token_driver.cu).  After the prompt and
    after every step the logits rows must agree within 2^-4 of the row's largest magnitude (bf16 roundings
    in another summation order, carried through 16 blocks) and the greedy token must be the same wherever
    the reference's two largest logits are further apart than twice the row's error."""
    root = os.path.dirname(REF_DIR.rstrip("/"))
    repo = os.path.dirname(root)
    cmds = {"ref": os.path.join(REF_DIR, "token_forward_ref")}
    for name, define in (("entry", "-DPA_SHIM"), ("classes", "-DPA_SHIM_CLASS")):
        exe = tmp_path / ("token_forward_" + name)
        r = subprocess.run(["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
                            define, "-I", os.path.join(repo, "include"), "-o", str(exe),
                            os.path.join(root, "token_driver.cu"),
                            "-L", os.path.join(repo, "llama_transformer_runtime_b200"), "-lpaged_attention",
                            "-Xlinker", "-rpath", "-Xlinker", os.path.join(repo, "llama_transformer_runtime_b200")],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-3000:]
        cmds[name] = str(exe)
    vocab, records = 128256, 13
    rec = np.dtype([("logits", np.uint16, (vocab,)), ("token", np.int32)])
    outs = {}
    for name, cmd in cmds.items():
        path = tmp_path / (name + ".bin")
        r = subprocess.run([cmd, str(path)], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, name + ": " + r.stdout[-2000:] + r.stderr[-2000:]
        outs[name] = np.fromfile(path, dtype=rec)
        assert outs[name].shape == (records,)
    for name in ("entry", "classes"):
        agree, same, report = 0, 0, []
        for s in range(records):
            g = orc.bf16_to_f32(outs[name]["logits"][s]).astype(np.float64)
            w = orc.bf16_to_f32(outs["ref"]["logits"][s]).astype(np.float64)
            assert np.isfinite(w).all() and np.isfinite(g).all()
            scale = np.abs(w).max()
            err = np.abs(g - w).max()
            assert scale > 0 and err <= 2.0 ** -4 * scale, f"{name}, record {s}: {err / scale}"
            # each program's token is the reference rule's answer on its own logits
            tok, ref_tok = int(outs[name]["token"][s]), int(outs["ref"]["token"][s])
            assert tok == int(orc.argmax_reference_rule(outs[name]["logits"][s:s + 1])[0])
            assert ref_tok == int(orc.argmax_reference_rule(outs["ref"]["logits"][s:s + 1])[0])
            top2 = np.partition(w, -2)[-2:]
            report.append((s, round(err / scale, 4), round((top2[1] - top2[0]) / scale, 4), tok, ref_tok))
            same += tok == ref_tok
            if top2[1] - top2[0] > 2 * err:
                assert tok == ref_tok, f"{name}, record {s}"
                agree += 1
        print(name, "record, max error / row max, (largest - second) / row max, token here, token of the reference:", report)
        assert agree >= records // 3, f"{name}: too few records with a clear winner to compare tokens: {report}"
        assert same >= records - 3, f"{name}: {report}"
