"""The vLLM sampler hook: `_fast_path_ok`, `_make_seeds`, `install_fused_sampler` and
`FusedSampler.sample`.

The CPU part drives the predicate with stand-in metadata objects (it only reads attributes).
The GPU part follows the reference's own tests of the hook
(tests/test_fused_sampler_predicate.py:18-197): a hand-built vLLM `SamplingMetadata`, the
patch installed and a subclass of upstream, greedy == upstream, processed-logprobs and
per-request generators fall back, top-k membership through the wrapper - plus top-p, which
this build keeps on the fast path.
"""

from types import SimpleNamespace

import numpy as np
import pytest
import torch


# --------------------------------------------------------------------------- CPU: predicate
def _meta(**kw):
    base = dict(allowed_token_ids_mask=None, bad_words_token_ids={},
                logitsprocs=SimpleNamespace(argmax_invariant=[], non_argmax_invariant=[]),
                thinking_budget_state_holder=None, generators={})
    base.update(kw)
    return SimpleNamespace(**base)


def test_fast_path_predicate_follows_the_reference():
    """reference _sampler.py:28-59: every feature outside the kernel sends the batch upstream."""
    from vllm_quant_kernels._sampler import _fast_path_ok
    assert _fast_path_ok(_meta())
    assert not _fast_path_ok(_meta(allowed_token_ids_mask=torch.zeros(2, 8, dtype=torch.bool)))
    assert not _fast_path_ok(_meta(bad_words_token_ids={0: [[3]]}))
    assert not _fast_path_ok(_meta(logitsprocs=SimpleNamespace(argmax_invariant=[object()], non_argmax_invariant=[])))
    assert not _fast_path_ok(_meta(logitsprocs=SimpleNamespace(argmax_invariant=[], non_argmax_invariant=[object()])))
    assert not _fast_path_ok(_meta(generators={0: object()}))
    busy = SimpleNamespace(has_tracked_requests=lambda: True)
    idle = SimpleNamespace(has_tracked_requests=lambda: False)
    assert not _fast_path_ok(_meta(thinking_budget_state_holder=busy))
    assert _fast_path_ok(_meta(thinking_budget_state_holder=idle))
    # a vLLM without the thinking-budget field at all
    m = _meta()
    del m.thinking_budget_state_holder
    assert _fast_path_ok(m)


def test_env_bool_truthy_set(monkeypatch):
    from vllm_quant_kernels._sampler import env_bool
    for v in ("1", "true", "YES", "On"):
        monkeypatch.setenv("VQK_TEST_FLAG", v)
        assert env_bool("VQK_TEST_FLAG")
    for v in ("0", "no", "off", "2"):
        monkeypatch.setenv("VQK_TEST_FLAG", v)
        assert not env_bool("VQK_TEST_FLAG")
    monkeypatch.delenv("VQK_TEST_FLAG")
    assert env_bool("VQK_TEST_FLAG", default=True) and not env_bool("VQK_TEST_FLAG")


# --------------------------------------------------------------------------- GPU: the hook
def _make_sampling_metadata(B, V, *, all_greedy=False, top_p=None, top_k=None, generators=None,
                            max_num_logprobs=None, temperature=None):
    from vllm.v1.sample.logits_processor.state import LogitsProcessors
    from vllm.v1.sample.metadata import SamplingMetadata
    if temperature is None:
        temperature = torch.zeros(B) if all_greedy else torch.ones(B)
    zeros = torch.zeros(B, dtype=torch.float32, device="cuda")
    return SamplingMetadata(
        temperature=temperature.to(torch.float32).cuda(), all_greedy=all_greedy, all_random=not all_greedy,
        top_p=top_p, top_k=top_k, generators=generators or {}, max_num_logprobs=max_num_logprobs,
        no_penalties=True, prompt_token_ids=None, frequency_penalties=zeros, presence_penalties=zeros,
        repetition_penalties=zeros + 1, output_token_ids=[[] for _ in range(B)], allowed_token_ids_mask=None,
        bad_words_token_ids={}, logitsprocs=LogitsProcessors(), logprob_token_ids=None, spec_token_ids=None,
        thinking_budget_state_holder=None)


@pytest.fixture
def fused_sampler_class():
    import vllm.v1.sample.sampler as upstream
    from vllm_quant_kernels._sampler import install_fused_sampler
    original = upstream.Sampler
    install_fused_sampler()
    yield upstream.Sampler, original
    upstream.Sampler = original


@pytest.mark.gpu
def test_install_replaces_sampler_with_a_subclass(fused_sampler_class):
    import vllm.v1.sample.sampler as upstream
    fused, original = fused_sampler_class
    assert upstream.Sampler is fused and fused.__name__ == "FusedSampler"
    assert issubclass(fused, original)
    s = fused()
    for name in ("compute_logprobs", "gather_logprobs", "apply_temperature"):
        assert hasattr(s, name)


@pytest.mark.gpu
def test_all_greedy_equals_upstream_argmax(fused_sampler_class):
    fused, original = fused_sampler_class
    B, V = 8, 4096
    logits = torch.randn(B, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(101))
    sm = _make_sampling_metadata(B, V, all_greedy=True)
    tok, processed = fused().sample(logits.clone(), sm)
    up, _ = original().sample(logits.clone(), sm)
    assert processed is None and tok.shape == (B,)
    assert torch.equal(tok.long(), logits.argmax(-1)) and torch.equal(tok.long(), up.long())


@pytest.mark.gpu
def test_random_rows_spread_and_mixed_greedy_rows_are_argmax(fused_sampler_class):
    fused, _ = fused_sampler_class
    B, V = 64, 256
    one = torch.randn(V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(202))
    logits = one.unsqueeze(0).expand(B, V).contiguous()
    T = torch.ones(B)
    T[:4] = 0.0                                            # mixed batch: four greedy rows
    sm = _make_sampling_metadata(B, V, temperature=T)
    tok, _ = fused().sample(logits.clone(), sm)
    assert tok.dtype == torch.int64 and (tok >= 0).all() and (tok < V).all()
    assert (tok[:4] == one.argmax()).all()
    assert len(set(tok[4:].tolist())) >= 5


@pytest.mark.gpu
def test_processed_logprobs_and_generators_fall_back_to_upstream(fused_sampler_class, monkeypatch):
    from vllm_quant_kernels import _sampler
    fused, _ = fused_sampler_class
    B, V = 4, 4096
    logits = torch.randn(B, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(404))
    calls = []
    monkeypatch.setattr(_sampler, "sample_logits", lambda *a, **k: calls.append(1) or (_ for _ in ()).throw(AssertionError))
    sm = _make_sampling_metadata(B, V, max_num_logprobs=5)
    tok, processed = fused(logprobs_mode="processed_logprobs").sample(logits.clone(), sm)
    assert tok.shape == (B,) and not calls
    gen = torch.Generator(device="cuda").manual_seed(42)
    sm = _make_sampling_metadata(B, V, generators={0: gen})
    tok, _ = fused().sample(logits.clone(), sm)
    assert tok.shape == (B,) and not calls


@pytest.mark.gpu
def test_raw_logprobs_request_stays_on_the_fast_path(fused_sampler_class, monkeypatch):
    """max_num_logprobs with the default raw_logprobs mode does not need processed logits."""
    from vllm_quant_kernels import _sampler
    fused, _ = fused_sampler_class
    B, V = 4, 4096
    logits = torch.randn(B, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    real = _sampler.sample_logits
    calls = []
    monkeypatch.setattr(_sampler, "sample_logits", lambda *a, **k: calls.append(1) or real(*a, **k))
    tok, processed = fused().sample(logits.clone(), _make_sampling_metadata(B, V, max_num_logprobs=5))
    assert calls and processed is None and tok.shape == (B,)


@pytest.mark.gpu
def test_top_k_and_top_p_membership_through_the_wrapper(fused_sampler_class):
    fused, _ = fused_sampler_class
    B, V, k = 8, 4096, 10
    logits = torch.randn(B, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(606)) * 3
    top_k = torch.full((B,), k, dtype=torch.int32, device="cuda")
    top_k[-1] = V                                          # vLLM's "disabled" for one row
    member = logits.topk(k, -1).indices
    for rep in range(4):
        tok, _ = fused().sample(logits.clone(), _make_sampling_metadata(B, V, top_k=top_k))
        assert (member[:-1] == tok[:-1, None]).any(-1).all()
    # top-p alone (the reference sent this upstream; here it runs in the CUDA sampler): the token
    # must lie in vLLM's own nucleus
    from vllm.v1.sample.ops.topk_topp_sampler import apply_top_k_top_p_pytorch
    p = torch.full((B,), 0.6, dtype=torch.float32, device="cuda")
    masked = apply_top_k_top_p_pytorch(logits.clone(), None, p)
    allowed = torch.isfinite(masked)
    for rep in range(4):
        tok, _ = fused().sample(logits.clone(), _make_sampling_metadata(B, V, top_p=p))
        assert allowed[torch.arange(B), tok].all()
    # both
    masked = apply_top_k_top_p_pytorch(logits.clone(), top_k.long(), p)
    allowed = torch.isfinite(masked)
    tok, _ = fused().sample(logits.clone(), _make_sampling_metadata(B, V, top_k=top_k, top_p=p))
    assert allowed[torch.arange(B), tok].all()


@pytest.mark.gpu
def test_make_seeds_follows_the_default_cuda_generator():
    """reference _sampler.py:96-116: int32 in [0, 2^31 - 1), one per row, from torch's default
    CUDA generator, so torch.manual_seed reproduces a run."""
    from vllm_quant_kernels._sampler import _make_seeds
    dev = torch.device("cuda", 0)
    torch.manual_seed(7)
    a = _make_seeds(33, dev)
    torch.manual_seed(7)
    b = _make_seeds(33, dev)
    c = _make_seeds(33, dev)
    assert a.dtype == torch.int32 and a.shape == (33,) and a.is_cuda
    assert torch.equal(a, b) and not torch.equal(b, c)
    assert int(a.min()) >= 0 and int(a.max()) < 2**31 - 1


@pytest.mark.gpu
def test_topk_threshold_wrapper_matches_torch_topk():
    """reference _sampler.py:62-93, without its host sync; disabled rows give -inf."""
    from vllm_quant_kernels._sampler import _compute_topk_threshold
    B, V = 6, 10000
    logits = torch.randn(B, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    k = torch.tensor([1, 5, 50, 400, V, 0], dtype=torch.int32, device="cuda")
    thr = _compute_topk_threshold(logits, k, V)
    for i, ki in enumerate(k.tolist()):
        want = logits[i].topk(ki).values[-1].item() if 0 < ki < V else -np.inf
        assert thr[i].item() == want


@pytest.mark.gpu
def test_try_fused_step_equals_the_two_hooks(monkeypatch):
    """`try_fused_step` (lm_head + sampler in one pass) against what the two plugin hooks give on
    the same inputs: `_quantized_forward` -> fp32 cast -> the CUDA sampler, same seeds."""
    from types import SimpleNamespace
    from tests.util import make_act, make_weight
    from vllm_quant_kernels import _lmhead as LH
    from vllm_quant_kernels._quant import QuantizedLogitsProcessor
    from vllm_quant_kernels._sampler import try_fused_step

    class FakeWeight:
        def __init__(self, t):
            self.data, self.dtype, self.shape, self.device = t, t.dtype, t.shape, t.device
    V, H, B = 100_016, 256, 6
    w = make_weight(V, H, seed=71) * 8.0
    x = make_act(B, H, seed=72)
    for e in ("VLLM_USE_W8A8_LMHEAD", "VLLM_USE_FP8_LMHEAD", "VLLM_USE_MXFP8_LMHEAD", "VLLM_USE_MXFP4_LMHEAD"):
        monkeypatch.delenv(e, raising=False)
    lm = SimpleNamespace(weight=FakeWeight(w))
    proc = QuantizedLogitsProcessor.__new__(QuantizedLogitsProcessor)
    proc.soft_cap, proc.scale, proc.logits_as_input, proc.org_vocab_size = 25.0, 1.0, False, V - 16
    seeds = torch.arange(B, dtype=torch.int32, device="cuda") + 100
    T = torch.tensor([0.0, 0.7, 0.9, 1.0, 1.2, 1.4])
    top_k = torch.tensor([50, 50, 10, V, 5, 50], dtype=torch.int32, device="cuda")
    top_p = torch.tensor([0.9, 0.9, 1.0, 0.8, 0.95, 0.5], dtype=torch.float32, device="cuda")
    sm = _make_sampling_metadata(B, V, temperature=T, top_k=top_k, top_p=top_p)
    sm.all_random = False
    tok = try_fused_step(proc, lm, x, sm, seeds=seeds)
    assert tok is not None and tok.dtype == torch.int64 and tok.shape == (B,)
    logits = proc.forward(lm, x).to(torch.float32)                    # soft-capped, padding trimmed
    assert logits.shape == (B, V - 16)
    want, _ = LH.sample_logits(logits, LH.SamplingArgs(T.cuda(), seeds, top_k, top_p))
    assert torch.equal(tok, want)
    assert tok[0] == logits[0].argmax()
    # off the fused path: logprobs wanted, penalties, a generator -> None (the runner falls back)
    assert try_fused_step(proc, lm, x, _make_sampling_metadata(B, V, temperature=T, max_num_logprobs=3)) is None
    sm2 = _make_sampling_metadata(B, V, temperature=T)
    sm2.no_penalties = False
    assert try_fused_step(proc, lm, x, sm2) is None
    gen = torch.Generator(device="cuda").manual_seed(1)
    assert try_fused_step(proc, lm, x, _make_sampling_metadata(B, V, temperature=T, generators={0: gen})) is None
    # all greedy
    tok = try_fused_step(proc, lm, x, _make_sampling_metadata(B, V, all_greedy=True))
    assert torch.equal(tok, logits.argmax(-1))
