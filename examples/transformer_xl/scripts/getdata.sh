#!/bin/bash
# Fetches and unpacks the corpora the run scripts expect under examples/transformer_xl/data/.
# Needs network access (there is none on the build box: the synthetic corpus of
# run_synthetic_moe.sh needs no download).
# usage: getdata.sh [enwik8] [text8] [wt103] [lm1b]      (default: all four)
set -e
cd "$(dirname "$0")/.."
mkdir -p data && cd data
want=${@:-enwik8 text8 wt103 lm1b}
for name in $want; do
  case $name in
    enwik8)
      mkdir -p enwik8 && cd enwik8
      [ -f enwik8.zip ] || wget -c http://mattmahoney.net/dc/enwik8.zip
      python - <<'PY'
import zipfile
data = zipfile.ZipFile("enwik8.zip").read("enwik8")
n = 5000000                                   # the customary 90M / 5M / 5M byte split
for split, part in (("train", data[:-2 * n]), ("valid", data[-2 * n:-n]), ("test", data[-n:])):
    with open(split + ".txt", "w") as f:
        f.write(" ".join(str(c) if c != ord("\n") else "\n" for c in part))
PY
      cd .. ;;
    text8)
      mkdir -p text8 && cd text8
      [ -f text8.zip ] || wget -c http://mattmahoney.net/dc/text8.zip
      python - <<'PY'
import zipfile
data = zipfile.ZipFile("text8.zip").read("text8").decode()
n = 5000000
for split, part in (("train", data[:-2 * n]), ("valid", data[-2 * n:-n]), ("test", data[-n:])):
    with open(split + ".txt", "w") as f:
        f.write(" ".join("_" if c == " " else c for c in part.strip()))
PY
      cd .. ;;
    wt103)
      [ -f wikitext-103-v1.zip ] || wget -c https://s3.amazonaws.com/research.metamind.io/wikitext/wikitext-103-v1.zip
      unzip -q -o wikitext-103-v1.zip ;;   # keeps wiki.{train,valid,test}.tokens, as the loader expects
    lm1b)
      mkdir -p one-billion-words && cd one-billion-words
      [ -f 1-billion-word-language-modeling-benchmark-r13output.tar.gz ] || \
        wget -c http://www.statmt.org/lm-benchmark/1-billion-word-language-modeling-benchmark-r13output.tar.gz
      tar xzf 1-billion-word-language-modeling-benchmark-r13output.tar.gz
      [ -f 1b_word_vocab.txt ] || wget -c https://github.com/rafaljozefowicz/lm/raw/master/1b_word_vocab.txt
      cd .. ;;
    *) echo "unknown corpus: $name" >&2; exit 1 ;;
  esac
done
