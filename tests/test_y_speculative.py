"""Speculative decoding over the MoE stack: one cheap draft layer proposes three tokens, the verify step runs the four
positions as ONE batch per layer through wd_moe_forward (the batch kernel), and the accepted tokens must be exactly the
tokens of plain greedy decoding, 64 out of 64 (the reference's MTP loop: draft_batched / verify,
src/qwen38_mtp.cuh:704-930). The glue between the blocks (RMSNorm, residual add, embedding, head) is the oracle's on
the host in both runs, so the only difference between them is one-token calls against four-token batches."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
H, F, E, K, SF, L, V = 512, 256, 32, 4, 256, 3, 512


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def test_speculative_decode_equals_plain_greedy(wd, oracle):
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(4242))
    ms = [synth.make_moe_block(5200 + l, H, F, E, K, SF) for l in range(L)]
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    embed = rng.standard_normal((V, H)).astype(np.float32)
    head = (rng.standard_normal((V, H)) * 0.05).astype(np.float32)
    eng = wd.Engine(H, F, E, K, SF, L, max_tokens=4)
    for l in range(L):
        eng.load_block(l, ms[l])

    def stack(tokens, layers):
        """next-token logits for every token of `tokens` (independent positions: the stack has no mixer), the MoE blocks
        of `layers` applied to all of them in one call per layer"""
        res = embed[np.asarray(tokens)].copy()
        for l in layers:
            x = np.stack([oracle.rmsnorm(r, norms[l], 1e-6) for r in res])
            out = eng.forward_host(l, x if len(tokens) > 1 else x[0]).reshape(len(tokens), H)
            res = (res + out).astype(np.float32)
        return res @ head.T

    n_tokens = 64
    # plain greedy: one token per step, one-token calls
    plain, tok = [], 17
    for _ in range(n_tokens):
        tok = int(np.argmax(stack([tok], range(L))[0]))
        plain.append(tok)
    # speculative: the draft is the first layer alone; verify runs the four positions as one batch per layer
    spec, tok, steps, accepted = [], 17, 0, 0
    while len(spec) < n_tokens:
        drafts, t = [], tok
        for _ in range(3):
            t = int(np.argmax(stack([t], [0])[0]))
            drafts.append(t)
        logits = stack([tok] + drafts, range(L))
        assert eng.last_kernel_name() == "moe_batch_kernel"
        nxt = [int(np.argmax(row)) for row in logits]
        spec.append(nxt[0])                     # the token after `tok` is always gained
        for i in range(3):
            if drafts[i] != nxt[i] or len(spec) >= n_tokens:
                break
            spec.append(nxt[i + 1])             # draft i was right: the token after it is valid too
            accepted += 1
        tok = spec[-1]
        steps += 1
    assert spec[:n_tokens] == plain             # 64 / 64
    assert len(set(plain)) > 8
    assert steps <= n_tokens and eng.device_status() == 0
    print("verify steps", steps, "accepted drafts", accepted)
    eng.close()
