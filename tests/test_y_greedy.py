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


def test_greedy_64_tokens_at_the_model_shape_with_the_full_head(wd, oracle):
    """Four layers of the 48-layer model's block shape (hidden 2048, 512 IQ3_S experts, top-10, Q8_0 shared expert),
    generated on the device, an embedding table and a Q8_0 output head over all 151,936 rows: 64 greedy tokens
    decoded on the device (embedding row -> stack -> head -> arg-max, nothing in the loop synchronises with the host)
    must agree 64/64 with the oracle chain on the same bytes, and so must the final residual bits."""
    import torch
    Hm, Fm, Em, Km, SFm, Lm, Vm = 2048, 512, 512, 10, 512, 4, 151936
    seed, n_tokens = 53, 64
    eng = wd.Engine(Hm, Fm, Em, Km, SFm, Lm)
    eng.synth_model(seed, 0.02, 0.0)
    rng = np.random.Generator(np.random.PCG64(54))
    norms = [(1.0 + 0.1 * rng.standard_normal(Hm)).astype(np.float32) for _ in range(Lm)]
    for l in range(Lm):
        eng.set_norm(l, norms[l])
    nb = Hm // 32
    table = torch.empty(Vm * nb * 34, dtype=torch.uint8, device="cuda")
    head_w = torch.empty(Vm * nb * 34, dtype=torch.uint8, device="cuda")
    wd.synth_tensor_device(wd.TYPE_Q8_0, Vm, Hm, 1.0, seed, 2000, table.data_ptr())
    wd.synth_tensor_device(wd.TYPE_Q8_0, Vm, Hm, 0.02, seed, 2001, head_w.data_ptr())
    torch.cuda.synchronize()
    head = wd.HeadQ8_0(Vm, Hm, ggml_dev_ptr=head_w.data_ptr())
    table_h = table.cpu().numpy().reshape(Vm, nb * 34)
    head_h = head_w.cpu().numpy()
    token = torch.tensor([4242], dtype=torch.int32, device="cuda")
    residual = torch.zeros(Hm, dtype=torch.float32, device="cuda")
    got = torch.zeros(n_tokens, dtype=torch.int32, device="cuda")
    ts = torch.cuda.Stream()
    stream = ts.cuda_stream
    with torch.cuda.stream(ts):
        for t in range(n_tokens):
            wd.embed_q8_0(table.data_ptr(), Vm, Hm, token.data_ptr(), residual.data_ptr(), stream)
            eng.stack_step_device(residual.data_ptr(), stream)
            head.argmax(residual.data_ptr(), token.data_ptr(), None, None, stream)
            got[t:t + 1].copy_(token)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    got = got.cpu().numpy().tolist()
    # the oracle chain; an expert's bytes are fetched when a token first selects it
    from warpdecode_b200 import synth
    dense = [eng.synth_dense_host(seed, 0.02, 0.0, l) for l in range(Lm)]
    gb = Fm * (Hm // 256) * 110
    weights = [[np.zeros(Em * gb, np.uint8) for _ in range(3)] for _ in range(Lm)]
    have = [set() for _ in range(Lm)]
    rb = nb * 34
    tok, want, res = 4242, [], None
    for t in range(n_tokens):
        res = synth.dequantize(ol.TYPE_Q8_0, table_h[tok], 1, Hm).reshape(Hm).astype(np.float32)
        for l in range(Lm):
            x = oracle.rmsnorm(res, norms[l], 1e-6)
            xq = oracle.quantize_q8_0(x)
            _, logits = oracle.head_argmax_q8_0(dense[l]["router"], Em, Hm, xq, logits=True)
            _, ids, _ = oracle.router(logits, Km, 1.0)
            for e in map(int, ids):
                if e not in have[l]:
                    g, u, d = eng.synth_expert_host(seed, 0.02, l, e)
                    for arr, src in zip(weights[l], (g, u, d)):
                        arr[e * gb:(e + 1) * gb] = src
                    have[l].add(e)
            m = dict(hidden=Hm, expert_ffn=Fm, shared_ffn=SFm, n_experts=Em, top_k=Km, gate_type=21, up_type=21, down_type=21,
                     w_scale=1.0, gate=weights[l][0], up=weights[l][1], down=weights[l][2], **dense[l])
            res = (res + oracle.moe_block(m, x)["out"]).astype(np.float32)
        tok = oracle.head_argmax_q8_0(head_h, Vm, Hm, oracle.quantize_q8_0(res))
        want.append(tok)
    assert got == want                                            # 64 / 64
    assert len(set(want)) > 8
    assert np.array_equal(bits(residual.cpu().numpy()), bits(res))
    head.close()
    eng.close()
