"""Greedy decode of a small MoE-stack model, token by token on the device (embedding row -> layers with
RMSNorm prologue and residual update -> Q8_0 head -> arg-max), against the same chain through the oracle:
every one of 64 tokens must agree, and so must the final residual bits."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
H, F, E, K, SF, L, V = 512, 256, 32, 4, 256, 3, 2048


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def test_greedy_64_tokens_agree_with_the_oracle_chain(wd, oracle):
    import torch
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(1234))
    ms = [synth.make_moe_block(1300 + l, H, F, E, K, SF) for l in range(L)]
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    embed = synth.quantize_q8_0(rng.standard_normal((V, H)).astype(np.float32)).reshape(V, -1)      # [V][H/32*34]
    head_w = synth.quantize_q8_0((rng.standard_normal((V, H)) * 0.05).astype(np.float32)).reshape(-1)
    eng = wd.Engine(H, F, E, K, SF, L)
    for l in range(L):
        eng.load_block(l, ms[l])
        eng.set_norm(l, norms[l])
    head = wd.HeadQ8_0(V, H, ggml_host=head_w)
    embed_dev = torch.from_numpy(embed.reshape(-1)).cuda()
    token = torch.tensor([17], dtype=torch.int32, device="cuda")
    residual = torch.zeros(H, dtype=torch.float32, device="cuda")
    n_tokens = 64
    got = torch.zeros(n_tokens, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    # one explicit stream for everything (a NULL stream would mean "the engine's own stream" to the engine)
    ts = torch.cuda.Stream()
    stream = ts.cuda_stream
    with torch.cuda.stream(ts):
        for t in range(n_tokens):          # nothing in this loop synchronises with the host
            wd.embed_q8_0(embed_dev.data_ptr(), V, H, token.data_ptr(), residual.data_ptr(), stream)
            eng.stack_step_device(residual.data_ptr(), stream)
            head.argmax(residual.data_ptr(), token.data_ptr(), None, None, stream)
            got[t:t + 1].copy_(token)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    got = got.cpu().numpy()
    # the oracle chain
    rb = H // 32 * 34
    tok, want = 17, []
    for t in range(n_tokens):
        res = synth.dequantize(ol.TYPE_Q8_0, embed[tok], 1, H).reshape(H).astype(np.float32)
        for l in range(L):
            x = oracle.rmsnorm(res, norms[l], 1e-6)
            res = (res + oracle.moe_block(ms[l], x)["out"]).astype(np.float32)
        xq = oracle.quantize_q8_0(res)
        logits = np.array([oracle.row(ol.TYPE_Q8_0, head_w[r * rb:(r + 1) * rb], xq, H) for r in range(V)], np.float32)
        finite = np.where(np.isfinite(logits), logits, -np.inf)
        tok = int(np.argmax(finite))        # numpy's argmax returns the first maximum: the lowest index
        want.append(tok)
    assert got.tolist() == want                                   # 64 / 64
    assert len(set(want)) > 8                                     # the sequence is not a fixed point
    assert np.array_equal(bits(residual.cpu().numpy()), bits(res))
    head.close()
    eng.close()
