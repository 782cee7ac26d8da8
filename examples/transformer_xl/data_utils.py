r"""
Corpora, vocabulary and batch iterators for the Transformer-XL example.

Counterpart of the reference's ``examples/transformer-xl/data_utils.py`` and
``utils/vocabulary.py``: word-level corpora with an ``<eos>`` per line (``ptb``, ``wt2``,
``wt103``), the sharded One Billion Word corpus with its published vocabulary (``lm1b``),
character-level corpora stored as space-separated symbols (``enwik8``, ``text8``),
contiguous batching for truncated back-propagation through time with an optional extended
context, an optional variable target length, and a binary cache next to the text files.
``synthetic`` needs no files: a Zipf-distributed token stream of a given vocabulary size.
"""
import os
from collections import Counter

import torch


class Vocab:
    r"""Symbol ↔ id map built from token counts (most frequent first)."""

    def __init__(self, special=(), min_freq=0, max_size=None, lower_case=False, delimiter=None):
        self.counter = Counter()
        self.special = list(special)
        self.min_freq, self.max_size = min_freq, max_size
        self.lower_case, self.delimiter = lower_case, delimiter
        self.idx2sym, self.sym2idx = [], {}

    def tokenize(self, line, add_eos=False):
        line = line.strip()
        if self.lower_case:
            line = line.lower()
        symbols = list(line) if self.delimiter == "" else line.split(self.delimiter)
        return symbols + ["<eos>"] if add_eos else symbols

    def count_file(self, path, add_eos=False):
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                self.counter.update(self.tokenize(line, add_eos))

    def _add(self, sym):
        if sym not in self.sym2idx:
            self.sym2idx[sym] = len(self.idx2sym)
            self.idx2sym.append(sym)

    def build(self):
        self.idx2sym, self.sym2idx = [], {}
        for sym in self.special:
            self._add(sym)
        for sym, cnt in self.counter.most_common(self.max_size):
            if cnt < self.min_freq:
                break
            self._add(sym)
        if "<unk>" in self.sym2idx:
            self.unk_idx = self.sym2idx["<unk>"]

    def index(self, sym):
        if sym in self.sym2idx:
            return self.sym2idx[sym]
        assert hasattr(self, "unk_idx"), "symbol %r is not in the vocabulary and there is no <unk>" % sym
        return self.unk_idx

    def encode_file(self, path, add_eos=True, sentence_marks=None):
        r"""Token ids of a text file.  ``sentence_marks``: a symbol put before and after every line
        (the One Billion Word corpus is a set of shuffled sentences, each wrapped in ``<S>``)."""
        ids = []
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                symbols = self.tokenize(line, add_eos)
                if sentence_marks is not None:
                    symbols = [sentence_marks] + symbols + [sentence_marks]
                ids.extend(self.index(s) for s in symbols)
        return torch.tensor(ids, dtype=torch.long)

    def build_from_file(self, path):
        r"""Vocabulary from a file with one symbol per line (first column), in file order."""
        self.idx2sym, self.sym2idx = [], {}
        for sym in self.special:
            self._add(sym)
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                parts = line.split()
                if parts:
                    self._add(parts[0])
        if "<UNK>" in self.sym2idx:
            self.unk_idx = self.sym2idx["<UNK>"]
        elif "<unk>" in self.sym2idx:
            self.unk_idx = self.sym2idx["<unk>"]

    def __len__(self):
        return len(self.idx2sym)


class LMOrderedIterator:
    r"""Splits one long token stream into ``bsz`` parallel streams and walks them in steps of
    ``bptt`` tokens, so that the hidden-state memory of batch ``i`` continues into batch ``i + 1``.

    Yields ``(data [ext_len + seq, bsz], target [seq, bsz], seq)``.
    """

    def __init__(self, data, bsz, bptt, device="cpu", ext_len=0, rank=0, world=1):
        self.bsz, self.bptt, self.ext_len, self.device = bsz, bptt, ext_len or 0, device
        n_step = data.numel() // (bsz * world)
        data = data[:n_step * bsz * world].view(bsz * world, n_step)
        # under data parallelism every rank walks its own bsz streams
        self.data = data[rank * bsz:(rank + 1) * bsz].t().contiguous()
        self.n_step = n_step
        self.n_batch = (n_step + bptt - 1) // bptt

    def get_batch(self, i, bptt=None):
        bptt = self.bptt if bptt is None else bptt
        seq = min(bptt, self.n_step - 1 - i)
        beg = max(0, i - self.ext_len)
        data = self.data[beg:i + seq].to(self.device, non_blocking=True)
        target = self.data[i + 1:i + 1 + seq].to(self.device, non_blocking=True)
        return data, target, seq

    def get_fixlen_iter(self, start=0):
        for i in range(start, self.n_step - 1, self.bptt):
            yield self.get_batch(i)

    def get_varlen_iter(self, start=0, std=5, min_len=5, max_deviation=3, generator=None):
        r"""Target length drawn around ``bptt`` (half of it with probability 0.05), as in AWD-LSTM."""
        max_len = self.bptt + max_deviation * std
        i = start
        while i < self.n_step - 2:
            base = self.bptt if torch.rand(1, generator=generator).item() < 0.95 else self.bptt / 2.0
            bptt = int(min(max_len, max(min_len, torch.normal(base, float(std), (1,), generator=generator).item())))
            data, target, seq = self.get_batch(i, bptt)
            i += seq
            yield data, target, seq

    def __iter__(self):
        return self.get_fixlen_iter()


class Corpus:
    r"""``train`` / ``valid`` / ``test`` token tensors plus the vocabulary."""

    WORD_LEVEL = ("ptb", "wt2", "wt103")
    CHAR_LEVEL = ("enwik8", "text8")

    def __init__(self, path, dataset, n_token=None, n_synthetic=2_000_000, seed=0):
        self.dataset = dataset
        if dataset == "synthetic":
            self.vocab = None
            self.n_token = int(n_token or 256)
            gen = torch.Generator().manual_seed(seed)
            weights = 1.0 / torch.arange(1, self.n_token + 1, dtype=torch.float64)
            stream = torch.multinomial(weights, n_synthetic, replacement=True, generator=gen)
            cut = n_synthetic // 20
            self.train, self.valid, self.test = stream[2 * cut:], stream[:cut], stream[cut:2 * cut]
            return
        if dataset in self.WORD_LEVEL:
            self.vocab = Vocab(special=["<eos>"], lower_case=(dataset == "wt103" and False))
            names = {"ptb": "ptb.%s.txt", "wt2": "wiki.%s.tokens", "wt103": "wiki.%s.tokens"}[dataset]
            add_eos = True
        elif dataset in self.CHAR_LEVEL:
            self.vocab = Vocab()
            names, add_eos = "%s.txt", False
        elif dataset == "lm1b":
            # One Billion Word: a published vocabulary file, 100 shuffled training shards and
            # 50 held-out shards (shard 0 is the customary validation / test set)
            import glob
            self.vocab = Vocab()
            self.vocab.build_from_file(os.path.join(path, "1b_word_vocab.txt"))
            root = os.path.join(path, "1-billion-word-language-modeling-benchmark-r13output")
            shards = sorted(glob.glob(os.path.join(root, "training-monolingual.tokenized.shuffled", "news.en-*")))
            held = os.path.join(root, "heldout-monolingual.tokenized.shuffled", "news.en.heldout-00000-of-00050")
            self.train = torch.cat([self.vocab.encode_file(f, add_eos=False, sentence_marks="<S>") for f in shards])
            self.valid = self.vocab.encode_file(held, add_eos=False, sentence_marks="<S>")
            self.test = self.valid
            self.n_token = len(self.vocab)
            return
        else:
            raise ValueError("unknown dataset %r" % dataset)
        files = {split: os.path.join(path, names % split) for split in ("train", "valid", "test")}
        self.vocab.count_file(files["train"], add_eos=add_eos)
        self.vocab.build()
        self.train = self.vocab.encode_file(files["train"], add_eos=add_eos)
        self.valid = self.vocab.encode_file(files["valid"], add_eos=add_eos)
        self.test = self.vocab.encode_file(files["test"], add_eos=add_eos)
        self.n_token = len(self.vocab)

    def get_iterator(self, split, bsz, bptt, device="cpu", ext_len=0, rank=0, world=1):
        return LMOrderedIterator(getattr(self, split), bsz, bptt, device=device, ext_len=ext_len,
                                 rank=rank, world=world)


def default_cutoffs(dataset, n_token):
    r"""Cluster boundaries of the adaptive softmax per corpus (frequency-sorted vocabulary)."""
    if dataset == "wt103":
        return [20000, 40000, 200000]
    if dataset == "lm1b":
        return [60000, 100000, 640000]
    if dataset == "synthetic" and n_token >= 4096:
        return [n_token // 16, n_token // 4]
    return []


def get_lm_corpus(path, dataset, **kwargs):
    r"""Loads ``<path>/cache.pt`` when present, otherwise builds the corpus and writes the cache."""
    if dataset == "synthetic":
        return Corpus(path, dataset, **kwargs)
    cache = os.path.join(path, "cache.pt")
    if os.path.exists(cache):
        return torch.load(cache, weights_only=False)
    corpus = Corpus(path, dataset, **kwargs)
    torch.save(corpus, cache)
    return corpus
