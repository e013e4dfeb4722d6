#!/usr/bin/env python3
"""
Create a Bliss lexicon whose "phonemes" are the BPE units: every word of a word list is segmented with the BPE codes and
written as a lemma with that pronunciation. (reference: tools/bpe-create-lexicon.py)
"""

import argparse
from xml.sax.saxutils import escape
import _setup_returnn_env  # noqa: F401
from returnn_b200.utils.bpe import StandardBytePairEncoder


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--bpe_codes", required=True)
    ap.add_argument("--bpe_vocab", required=True, help="Python dict {unit: index}")
    ap.add_argument("--words", required=True, help="one word per line (further columns are ignored)")
    ap.add_argument("--output", required=True)
    ap.add_argument("--unk", default="<unk>")
    args = ap.parse_args()
    vocab = eval(open(args.bpe_vocab).read())
    bpe = StandardBytePairEncoder(args.bpe_codes, labels=list(vocab.keys()))
    with open(args.output, "w", encoding="utf8") as out:
        out.write('<?xml version="1.0" encoding="utf-8"?>\n<lexicon>\n<phoneme-inventory>\n')
        for unit in sorted(vocab.keys(), key=lambda u: vocab[u]):
            out.write("<phoneme><symbol>%s</symbol></phoneme>\n" % escape(unit))
        out.write("</phoneme-inventory>\n")
        n = 0
        for line in open(args.words, encoding="utf8"):
            parts = line.split()
            if not parts:
                continue
            word = parts[0]
            units = bpe.segment_sentence(word)
            if any(u not in vocab for u in units):
                units = [args.unk]
            out.write("<lemma><orth>%s</orth><phon>%s</phon></lemma>\n" % (escape(word), escape(" ".join(units))))
            n += 1
        out.write("</lexicon>\n")
    print("wrote %i lemmas" % n)


if __name__ == "__main__":
    main()
