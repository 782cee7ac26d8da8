r"""CPU tests of the example-side model pieces: adaptive embedding / softmax, corpus iterators,
and a few optimisation steps of the Transformer-XL training script with checkpoint restart."""
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "transformer_xl"))
sys.path.insert(0, os.path.join(ROOT, "examples"))


def test_adaptive_softmax_is_a_distribution_and_matches_its_nll():
    from fastmoe_b200.models.adaptive import ProjectedAdaptiveLogSoftmax
    torch.manual_seed(0)
    for cutoffs, div_val in (((), 1), ((10, 30), 1), ((10, 30), 2), ((8,), 4)):
        crit = ProjectedAdaptiveLogSoftmax(50, 16, 16, cutoffs, div_val)
        for p in crit.parameters():
            if p.numel():
                torch.nn.init.normal_(p, 0.0, 0.3)
        hidden = torch.randn(40, 16)
        target = torch.randint(0, 50, (40,))
        logp = crit.log_prob(hidden)
        assert logp.shape == (40, 50)
        assert torch.allclose(torch.logsumexp(logp, dim=-1), torch.zeros(40), atol=1e-5)
        nll = crit(hidden, target)
        assert torch.allclose(nll, -logp.gather(1, target[:, None]).squeeze(1), atol=1e-5)


def test_adaptive_softmax_without_cutoffs_is_plain_cross_entropy():
    from fastmoe_b200.models.adaptive import ProjectedAdaptiveLogSoftmax
    torch.manual_seed(1)
    crit = ProjectedAdaptiveLogSoftmax(20, 8, 8)
    hidden, target = torch.randn(11, 8), torch.randint(0, 20, (11,))
    ref = torch.nn.functional.cross_entropy(
        torch.nn.functional.linear(hidden, crit.out_layers[0].weight, crit.out_layers[0].bias), target,
        reduction="none")
    assert torch.allclose(crit(hidden, target), ref, atol=1e-6)


def test_adaptive_embedding_and_weight_tying():
    from fastmoe_b200.models.adaptive import AdaptiveEmbedding, ProjectedAdaptiveLogSoftmax
    torch.manual_seed(2)
    emb = AdaptiveEmbedding(50, 16, 16, (10, 30), div_val=2)
    tokens = torch.tensor([[0, 9, 10], [29, 30, 49]])
    out = emb(tokens)
    assert out.shape == (2, 3, 16)
    # a shortlist token is its table row times sqrt(d_proj); a tail token goes through its projection
    assert torch.allclose(out[0, 1], emb.emb_layers[0].weight[9] * 4.0)
    want = torch.nn.functional.linear(emb.emb_layers[2].weight[19], emb.emb_projs[2]) * 4.0
    assert torch.allclose(out[1, 2], want, atol=1e-6)
    crit = ProjectedAdaptiveLogSoftmax(50, 16, 16, (10, 30), div_val=2)
    crit.tie_weights(emb, tie_projs=[False, True, True])
    assert crit.out_layers[1].weight is emb.emb_layers[1].weight
    assert crit.out_projs[2] is emb.emb_projs[2]
    assert crit.out_projs[0].numel() == 0


def test_ordered_iterator_streams_are_contiguous():
    from data_utils import Corpus, LMOrderedIterator
    data = torch.arange(1000)
    it = LMOrderedIterator(data, bsz=4, bptt=7, ext_len=2)
    batches = list(it)
    first, second = batches[0], batches[1]
    assert first[0].shape == (7, 4) and first[1].shape == (7, 4)
    assert torch.equal(first[1], first[0] + 1)                    # target is the next token
    assert torch.equal(second[0][2:], first[0][-1:] + 1 + torch.arange(7)[:, None])  # continues the stream
    assert second[0].shape[0] == 7 + 2                            # extended context
    total = sum(b[2] for b in batches)
    assert total == 1000 // 4 - 1
    # data-parallel ranks walk disjoint streams
    a = LMOrderedIterator(data, 2, 5, rank=0, world=2).data
    b = LMOrderedIterator(data, 2, 5, rank=1, world=2).data
    assert not set(a.flatten().tolist()) & set(b.flatten().tolist())
    corpus = Corpus(".", "synthetic", n_token=64, n_synthetic=20000)
    assert corpus.n_token == 64 and int(corpus.train.max()) < 64
    lengths = [seq for _, _, seq in corpus.get_iterator("valid", 2, 16).get_varlen_iter()]
    assert sum(lengths) >= 1000 // 2 - 20 and min(lengths) >= 1


def test_vocab_round_trip(tmp_path):
    from data_utils import Vocab
    text = tmp_path / "t.txt"
    text.write_text("a b b c\nb a\n")
    vocab = Vocab(special=["<eos>"])
    vocab.count_file(str(text), add_eos=True)
    vocab.build()
    ids = vocab.encode_file(str(text), add_eos=True)
    assert [vocab.idx2sym[i] for i in ids.tolist()] == ["a", "b", "b", "c", "<eos>", "b", "a", "<eos>"]
    assert vocab.idx2sym[1] == "b"        # most frequent non-special symbol first


def test_transformer_xl_training_script_learns_and_restarts(tmp_path, capsys):
    import train as xl_train
    common = ["--dataset", "synthetic", "--n_token", "5000", "--adaptive", "--div_val", "2", "--n_layer", "2",
              "--d_model", "32", "--n_head", "2", "--d_head", "16", "--d_inner", "64", "--tgt_len", "16",
              "--mem_len", "16", "--eval_tgt_len", "8", "--batch_size", "4", "--moe", "--moe-num-expert", "2",
              "--log-interval", "5", "--eval-interval", "10", "--max_eval_steps", "3", "--lr", "0.01",
              "--dropout", "0.0", "--work_dir", str(tmp_path)]
    xl_train.main(common + ["--max_step", "10"])
    first = capsys.readouterr().out
    losses = [float(line.split("| loss")[1].split("|")[0]) for line in first.splitlines() if "| loss" in line]
    assert len(losses) == 2 and losses[-1] < losses[0] and math.isfinite(losses[-1])
    assert "eval at step     10" in first
    assert os.path.exists(os.path.join(str(tmp_path), "latest"))
    xl_train.main(common + ["--max_step", "12", "--restart", "--batch_chunk", "2", "--scheduler", "inv_sqrt",
                            "--warmup_step", "2"])
    second = capsys.readouterr().out
    assert "| step     12 |" in second and "| step      5 |" not in second

    import eval as xl_eval
    loss = xl_eval.main(common + ["--split", "valid"])
    assert math.isfinite(loss)


def test_log_uniform_sampler_and_sampled_softmax():
    from fastmoe_b200.models.sampled_softmax import LogUniformSampler, sampled_softmax_nll
    sampler = LogUniformSampler(500, 40, torch.Generator().manual_seed(1))
    assert abs(float(sampler.prob.sum()) - 1.0) < 1e-9
    assert bool((sampler.prob[:-1] >= sampler.prob[1:]).all())       # frequent classes first
    labels = torch.randint(0, 500, (30,))
    true_q, samp_q, negatives = sampler.sample(labels)
    assert negatives.unique().numel() == negatives.numel() <= 80
    assert true_q.shape == (30,) and samp_q.shape == negatives.shape
    # with every class as a "negative" and no proposal correction the loss is the full softmax
    class Everything:
        def sample(self, lab):
            return torch.zeros(lab.shape[0]), torch.zeros(500), torch.arange(500)
    w, b, h = torch.randn(500, 8), torch.randn(500), torch.randn(30, 8)
    nll = sampled_softmax_nll(w, b, h, labels, Everything())
    ref = torch.nn.functional.cross_entropy(h @ w.t() + b, labels, reduction="none")
    assert torch.allclose(nll, ref, atol=1e-4)


def test_balanced_data_parallel_chunk_sizes(tmp_path):
    from exp_utils import balanced_chunk_sizes, create_exp_dir
    assert balanced_chunk_sizes(22, 4, 4) == [4, 6, 6, 6]
    assert balanced_chunk_sizes(22, 4, 0) == [0, 8, 7, 7]
    assert balanced_chunk_sizes(5, 4, 4) == [4, 1]
    assert balanced_chunk_sizes(8, 1, 2) == [8]
    log = create_exp_dir(str(tmp_path / "run"), scripts_to_save=[__file__])
    log("hello", print_=False)
    assert (tmp_path / "run" / "log.txt").read_text() == "hello\n"
    assert (tmp_path / "run" / "scripts" / os.path.basename(__file__)).exists()
