"""Samplers, logits processors, beam search and API behaviours on the CPU path (+ GPU kernels where marked)."""
import pytest
import torch

from xfastertransformer_b200.ops import reference as R
from xfastertransformer_b200.runtime import sampler as S
from xfastertransformer_b200.runtime.sequence import SamplingMeta


def test_repetition_penalty_rule():
    l = torch.tensor([[2.0, -2.0, 1.0, 0.5]])
    out = R.repetition_penalty(l.clone(), [[0, 1, 1, 9]], 2.0, 0)
    assert out.tolist() == [[1.0, -4.0, 1.0, 0.5]]
    # ids outside this rank's vocab slice are ignored
    out = R.repetition_penalty(l.clone(), [[4, 5]], 2.0, 4)
    assert out.tolist() == [[1.0, -4.0, 1.0, 0.5]]


def test_top_p_keeps_at_least_two():
    logits = torch.tensor([[10.0, 0.0, -1.0, -2.0]])
    picks = {int(R.sample_top_k_top_p(logits, 4, 0.01, 1.0, torch.tensor([u]))[0]) for u in (0.0, 0.5, 0.99999)}
    assert picks <= {0, 1} and 0 in picks


def test_stop_words_cleaning_and_matching():
    cfg = SamplingMeta(eos_token_id=2, stop_words=[[], [0, 3], [2], [5, 6], [7]])
    cfg.clean_stop_words()
    assert cfg.stop_words == [[5, 6], [7]]
    assert S.match_stop_words([1, 5, 6], cfg.stop_words)
    assert not S.match_stop_words([5, 6, 1], cfg.stop_words)


def test_beam_scorer_prefers_higher_logprob():
    cfg = SamplingMeta(num_beams=2, eos_token_id=3, pad_token_id=0, max_length=8)
    sc = S.BeamSearchScorer(1, cfg, 0)
    lp = torch.full((2, 5), -10.0)
    lp[0, 1] = -0.1
    lp[0, 2] = -0.5
    toks, src = sc.process(lp)
    assert toks.tolist() == [1, 2] and src.tolist() == [0, 0]
    lp = torch.full((2, 5), -10.0)
    lp[0, 3] = -0.05          # beam 0 ends with eos
    lp[1, 4] = -0.2
    toks, src = sc.process(lp)
    outs = sc.finalize([[9]], 8)
    assert outs[0][:3] == [9, 1, 3]


@pytest.mark.gpu
def test_gpu_sampler_matches_reference():
    from xfastertransformer_b200.ops import native_sample
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(9, 32000, generator=g) * 3
    for k, p, T in ((50, 0.9, 0.8), (1, 1.0, 1.0), (1024, 0.5, 1.3), (5, 1.0, 0.7)):
        u = torch.rand(9, generator=g)
        want = R.sample_top_k_top_p(logits, k, p, T, u)
        got = native_sample.sample_top_k_top_p(logits.cuda(), k, p, T, u).cpu()
        # identical except where the draw lands within float error of a CDF boundary
        assert (got == want).float().mean().item() >= 0.85, (k, p, T, got, want)
    # k outside [1, 1024] is clamped the same way on both sides (0 -> 1, above the candidate capacity -> 1024, V)
    small = torch.randn(5, 700, generator=g) * 2
    for k, src in ((0, logits), (-3, logits), (1, logits), (4000, logits), (700, small), (5000, small)):
        u = torch.rand(src.shape[0], generator=g)
        want = R.sample_top_k_top_p(src, k, 0.95, 1.0, u)
        got = native_sample.sample_top_k_top_p(src.cuda(), k, 0.95, 1.0, u).cpu()
        assert int(got.min()) >= 0 and int(got.max()) < src.shape[1]
        assert (got == want).float().mean().item() >= 0.8, (k, got, want)
    # ties: all-equal logits keep the k lowest indices, whatever the thread timing (every rank picks the same token)
    flat = torch.zeros(4, 5000)
    u = torch.tensor([0.0, 0.3, 0.6, 0.999])
    for k in (1, 7, 1024, 3000):
        got = native_sample.sample_top_k_top_p(flat.cuda(), k, 1.0, 1.0, u).cpu()
        kk = max(1, min(k, 1024))
        assert int(got.max()) < kk and got.tolist() == [min(kk - 1, int(x * kk)) for x in u.tolist()], (k, got)
        assert got.tolist() == native_sample.sample_top_k_top_p(flat.cuda(), k, 1.0, 1.0, u).cpu().tolist()
    l = torch.randn(3, 100)
    toks = [[1, 2, 2, 50], [], [99, 0]]
    want = R.repetition_penalty(l.clone(), toks, 1.7, 0)
    got = native_sample.repetition_penalty(l.clone().cuda(), toks, 1.7, 0).cpu()
    assert torch.allclose(got, want)


def test_beam_step_from_per_beam_topk_matches_full_vocabulary_step():
    """`process_topk` (each beam's 2 x beams best continuations) takes the same decisions as `process` (the whole
    vocabulary): tokens, source beams, running scores, finished hypotheses."""
    import copy
    from xfastertransformer_b200 import ops
    from xfastertransformer_b200.runtime.sampler import BeamSearchScorer
    from xfastertransformer_b200.runtime.sequence import SamplingMeta
    g = torch.Generator().manual_seed(5)
    for nb, V, eos in [(2, 50, 3), (4, 97, 0), (3, 5, 1)]:
        cfg = SamplingMeta(num_beams=nb, max_length=64, eos_token_id=eos, pad_token_id=0, length_penalty=1.0,
                           early_stopping=False)
        a = BeamSearchScorer(3, cfg, 0)
        b = copy.deepcopy(a)
        for step in range(6):
            logits = torch.randn(3 * nb, V, generator=g) * 3
            ta, sa = a.process(torch.log_softmax(logits, -1))
            tb, sb = b.process_topk(*ops.beam_topk(logits, min(2 * nb, V)))
            assert ta.tolist() == tb.tolist() and sa.tolist() == sb.tolist(), (nb, V, step)
            torch.testing.assert_close(a.beam_scores, b.beam_scores, rtol=1e-5, atol=1e-5)
            assert a.done == b.done and a.seqs == b.seqs
            assert [len(h.beams) for h in a.hyps] == [len(h.beams) for h in b.hyps]


def test_beam_topk_reference_orders_ties_by_token_id():
    from xfastertransformer_b200.ops import reference as R
    x = torch.tensor([[1.0, 3.0, 3.0, -2.0, 3.0, 0.5]])
    v, i = R.beam_topk(x, 4)
    assert i.tolist() == [[1, 2, 4, 0]]
    torch.testing.assert_close(v, torch.log_softmax(x, -1)[0, [1, 2, 4, 0]][None])


@pytest.mark.gpu
def test_gpu_beam_topk_matches_reference():
    """Device beam step: log-softmax and the k best entries of each row against the fp32 reference; rows with many
    equal logits come back in token-id order."""
    from xfastertransformer_b200.ops import native_sample, reference as R
    g = torch.Generator().manual_seed(11)
    for rows, V, k in [(6, 32000, 8), (3, 151936, 64), (4, 50, 2), (2, 7, 7), (5, 1025, 1)]:
        x = torch.randn(rows, V, generator=g) * 4
        wv, wi = R.beam_topk(x, k)
        gv, gi = native_sample.beam_topk(x.cuda(), k)
        torch.testing.assert_close(gv.cpu(), wv, rtol=1e-5, atol=2e-4)
        assert torch.equal(x.gather(1, gi.cpu()), x.gather(1, wi)), (rows, V, k)
    x = torch.randint(-3, 4, (4, 5000), generator=g).float()      # 7 distinct values: ties everywhere
    wv, wi = R.beam_topk(x, 16)
    gv, gi = native_sample.beam_topk(x.cuda(), 16)
    assert gi.cpu().tolist() == wi.tolist()
    torch.testing.assert_close(gv.cpu(), wv, rtol=1e-5, atol=2e-4)
    strided = torch.randn(3, 2 * 4096, generator=g).cuda()[:, :4096]      # a view with a row stride
    gv, gi = native_sample.beam_topk(strided, 6)
    wv, wi = R.beam_topk(strided.cpu(), 6)
    assert gi.cpu().tolist() == wi.tolist()


def test_beam_hypotheses_are_normalised_by_prompt_plus_generated_length():
    """The reference scores a finished hypothesis as sum of log-probabilities / (length of the whole row of ids) **
    length_penalty, the row being prompt + tokens generated before the closing one (src/searchers/beam_search.cpp:87-112,
    161-171).  With a long prompt the normalisation barely changes between a short and a long continuation, so the short
    one with the better sum wins; with no prompt the long one does."""
    from xfastertransformer_b200.runtime.sampler import BeamSearchScorer
    from xfastertransformer_b200.runtime.sequence import SamplingMeta
    V, eos = 6, 1
    cfg = SamplingMeta(num_beams=2, max_length=64, eos_token_id=eos, pad_token_id=0, length_penalty=1.0, early_stopping=False)

    def run(prompt_len):
        sc = BeamSearchScorer(1, cfg, prompt_len)
        neg = -30.0
        # step 1: beam 0 may stop (eos at -1.0) or go on with token 2 (-1.2); token 3 (-1.4) keeps a second beam alive
        lp = torch.full((2, V), neg)
        lp[0, eos], lp[0, 2], lp[0, 3] = -1.0, -1.2, -1.4
        sc.process(lp)
        # steps 2, 3: cheap continuations (token 4 at -0.1) for both beams, then the first beam closes cheaply
        for _ in range(2):
            lp = torch.full((2, V), neg)
            lp[:, 4] = -0.1
            sc.process(lp)
        lp = torch.full((2, V), neg)
        lp[0, eos], lp[0, 4], lp[1, 4] = -0.1, -5.0, -0.2
        sc.process(lp)
        return sc.hyps[0].beams

    short_first = sorted(run(100), key=lambda x: -x[0])
    long_first = sorted(run(0), key=lambda x: -x[0])
    # hypotheses: short = [eos] with sum -1.0, long = [2, 4, 4, eos] with sum -1.5
    assert short_first[0][1] == [eos] and abs(short_first[0][0] - (-1.0 / 100)) < 1e-6
    assert abs(short_first[1][0] - (-1.5 / 103)) < 1e-6
    assert long_first[0][1] == [2, 4, 4, eos] and abs(long_first[0][0] - (-1.5 / 3)) < 1e-6
    assert abs(long_first[1][0] - (-1.0 / 1)) < 1e-6
