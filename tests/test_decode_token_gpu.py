"""The whole decode step: pa_embedding and pa_decode_token (the body of the reference's
LlamaRuntime::decode_forward, src/runtime/llama_runtime.cu:822-945)."""
import numpy as np
import pytest
import torch

from llama_transformer_runtime_b200 import _lib, paged
from oracle import oracle as orc
from tests.gpu_helpers import DEV, f32_dev, to_dev, to_u16
from tests.test_attention_chain_gpu import _fill, _model
from tests.test_ffn_gpu import _ffn_model

pytestmark = pytest.mark.gpu

EPS = 1e-5


def test_embedding_rows_vs_table_and_reference(cuda):
    rng = np.random.default_rng(1300)
    vocab = 3000
    table = orc.randn_bf16(rng, (vocab, 2048), 1.0)
    ids = np.array([0, 2999, 17, 17, 1234], np.int32)
    td, idd = to_dev(table), torch.from_numpy(ids).to(DEV)
    out = torch.full((len(ids), 2048), 3.0, dtype=torch.bfloat16, device=DEV)
    paged.embedding(idd, td, out, len(ids))
    torch.cuda.synchronize()
    assert np.array_equal(to_u16(out), table[ids])
    if orc.ref_available():
        ref_out = torch.zeros_like(out)
        orc.ref().ref_embedding(idd.data_ptr(), td.data_ptr(), ref_out.data_ptr(), len(ids))
        torch.cuda.synchronize()
        assert np.array_equal(to_u16(out), to_u16(ref_out))
    # ids outside the table: a row of zeros, nothing read out of range
    bad = torch.tensor([5, -1, vocab], dtype=torch.int32, device=DEV)
    out3 = torch.full((3, 2048), 3.0, dtype=torch.bfloat16, device=DEV)
    paged.embedding(bad, td, out3, 3)
    torch.cuda.synchronize()
    got = to_u16(out3)
    assert np.array_equal(got[0], table[5]) and not got[1:].any()
    with pytest.raises(_lib.PagedAttentionError) as ei:
        paged.embedding(None, td, out3, 3)
    assert ei.value.code == 1


@pytest.mark.parametrize("lens", [[37], [300, 16, 95]])
def test_decode_token_equals_its_parts_and_the_reference_token_rule(cuda, lens):
    """Three steps of a 2-layer model with a 4096-entry vocabulary, each step's ids the previous step's
    output read on the device.  The same steps run as the separate calls (embedding, block step,
    language-model head, argmax — each checked against the oracle and the reference's kernels in its own
    test) must give the same logits bit for bit and the same tokens; every token must be the reference
    kernel's answer on those logits."""
    rng = np.random.default_rng(1310 + len(lens))
    layers, steps, n, vocab = 2, 3, len(lens), 4096
    nw, wq, wk, wv, wo = _model(rng, layers)
    fn, wg, wu, wd = _ffn_model(rng, layers)
    table = orc.randn_bf16(rng, (vocab, 2048), 1.0)
    final_norm = orc.randn_bf16(rng, (2048,), 0.7)
    w_lm = orc.randn_bf16(rng, (2048, vocab), 0.03)
    cos, sin = orc.build_rope_tables(max(lens) + steps + 1)
    cos_d, sin_d = f32_dev(cos), f32_dev(sin)
    nb = sum((L + steps + 15) // 16 for L in lens) + 8
    Ks = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    Vs = [[orc.randn_bf16(rng, (8, L + steps, 64), 0.5) for _ in range(layers)] for L in lens]
    first = rng.integers(0, vocab, n).astype(np.int32)
    results = []
    for mode in ("one_call", "parts"):
        pool = paged.KVPool(layers, nb, 8, n, max((L + steps + 15) // 16 for L in lens) + 1)
        pool.set_free_order(np.random.default_rng(3).permutation(nb))
        seqs = [pool.create_seq() for _ in lens]
        for i, L in enumerate(lens):
            _fill(pool, seqs[i], layers, Ks[i], Vs[i], L)
        at = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
        ft = [to_dev(a) for a in (fn, wg, wu, wd)]
        td, fd, ld = to_dev(table), to_dev(final_norm), to_dev(w_lm)
        WA, WF = paged.attention_weights(*at), paged.ffn_weights(*ft)
        M = paged.model_weights(td, WA, WF, fd, ld, EPS)
        tok = torch.from_numpy(first).to(DEV)
        logits = [torch.zeros(n, vocab, dtype=torch.bfloat16, device=DEV) for _ in range(steps)]
        toks = []
        for step in range(steps):
            for i in range(n):
                pool.reserve(seqs[i], lens[i] + step + 1)
            pool.batch_set(seqs, [1] * n)
            if mode == "one_call":
                paged.decode_token(pool, M, tok, tok, logits[step], cos_d, sin_d, chained=step > 0)
            else:
                x0 = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                x1 = torch.zeros(n, 2048, dtype=torch.bfloat16, device=DEV)
                paged.embedding(tok, td, x0, n)
                paged.block_step(pool, WA, WF, 0, layers, x0, x1, cos_d, sin_d)
                paged.lm_head(x1, fd, ld, logits[step], n, EPS)
                paged.argmax(logits[step], tok, n)
            toks.append(tok.clone())
        torch.cuda.synchronize()
        pool.check()
        results.append(([to_u16(l) for l in logits], [t.cpu().numpy() for t in toks]))
        pool.close()
    (lg_a, tk_a), (lg_b, tk_b) = results
    for step in range(steps):
        assert np.array_equal(lg_a[step], lg_b[step]), f"step {step}: logits differ from the separate calls"
        assert np.array_equal(tk_a[step], tk_b[step])
        assert np.array_equal(tk_a[step], orc.argmax_reference_rule(lg_a[step]))
        assert np.isfinite(orc.bf16_to_f32(lg_a[step])).all()


def test_decode_token_records_an_id_out_of_range(cuda):
    rng = np.random.default_rng(1320)
    layers, vocab = 1, 64
    nw, wq, wk, wv, wo = _model(rng, layers)
    fn, wg, wu, wd = _ffn_model(rng, layers)
    pool = paged.KVPool(layers, 4, 8, 1, 2)
    s = pool.create_seq()
    pool.reserve(s, 1)
    pool.batch_set([s], [1])
    at = [to_dev(a) for a in (nw, wq, wk, wv, wo)]
    ft = [to_dev(a) for a in (fn, wg, wu, wd)]
    td, ld = to_dev(orc.randn_bf16(rng, (vocab, 2048), 1.0)), to_dev(orc.randn_bf16(rng, (2048, vocab), 0.03))
    WA, WF = paged.attention_weights(*at), paged.ffn_weights(*ft)
    M = paged.model_weights(td, WA, WF, None, ld, EPS)
    cos, sin = orc.build_rope_tables(4)
    tok = torch.tensor([vocab + 3], dtype=torch.int32, device=DEV)
    out = torch.zeros(1, dtype=torch.int32, device=DEV)
    logits = torch.zeros(1, vocab, dtype=torch.bfloat16, device=DEV)
    paged.decode_token(pool, M, tok, out, logits, f32_dev(cos), f32_dev(sin))
    torch.cuda.synchronize()
    with pytest.raises(_lib.PagedAttentionError) as ei:
        pool.check()
    assert ei.value.code == 1
    pool.check()  # the word was cleared
    with pytest.raises(_lib.PagedAttentionError):
        paged.decode_token(pool, M, None, out, logits, f32_dev(cos), f32_dev(sin))
    pool.close()
