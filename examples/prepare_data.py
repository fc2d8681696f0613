"""Turn text into the flat token file that `lt.data.TokenStream` and examples/train_llama.py read.

    python examples/prepare_data.py --input corpus.txt --out tokens.bin                       # byte-level ids (0-255) + 256 = end of document
    python examples/prepare_data.py --input corpus.txt --out tokens.bin --sentencepiece tok.model
    python examples/prepare_data.py --input a.txt b.txt --out tokens.bin --dtype uint32

Documents are separated by blank lines; an end-of-document id follows each one (the tokenizer's EOS, or 256 at byte
level).  The file is written in pieces, so the corpus never has to fit in memory; a JSON side file records the
vocabulary size, the dtype and the token count.
"""
import argparse
import json
import os
import sys

import numpy as np


def documents(paths):
    for p in paths:
        doc = []
        with open(p, encoding="utf-8", errors="replace") as f:
            for line in f:
                if line.strip():
                    doc.append(line)
                elif doc:
                    yield "".join(doc)
                    doc = []
        if doc:
            yield "".join(doc)


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", nargs="+", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--sentencepiece", default="", help="a SentencePiece model file; default: byte-level ids")
    ap.add_argument("--dtype", default="uint16", choices=["uint16", "uint32"])
    args = ap.parse_args(argv)
    if args.sentencepiece:
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=args.sentencepiece)
        vocab, eos = sp.get_piece_size(), (sp.eos_id() if sp.eos_id() >= 0 else sp.get_piece_size() - 1)
        encode = lambda text: sp.encode(text)
    else:
        vocab, eos = 257, 256
        encode = lambda text: list(text.encode("utf-8"))
    dt = np.dtype(args.dtype)
    if vocab - 1 > np.iinfo(dt).max:
        sys.exit("vocabulary of %d does not fit %s" % (vocab, args.dtype))
    total = docs = 0
    tmp = args.out + ".tmp"
    with open(tmp, "wb") as out:
        buf = []
        for doc in documents(args.input):
            buf += encode(doc) + [eos]
            docs += 1
            if len(buf) >= 1 << 20:
                np.asarray(buf, dtype=dt).tofile(out)
                total += len(buf)
                buf = []
        np.asarray(buf, dtype=dt).tofile(out)
        total += len(buf)
    os.replace(tmp, args.out)
    meta = {"tokens": total, "documents": docs, "vocab_size": vocab, "eos_id": eos, "dtype": args.dtype,
            "tokenizer": args.sentencepiece or "bytes"}
    with open(args.out + ".json", "w") as f:
        json.dump(meta, f, indent=1)
    print(json.dumps(meta))
    return meta


if __name__ == "__main__":
    main()
