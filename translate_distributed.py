#!/usr/bin/env python
"""Data-parallel translation: the source file is split into one contiguous part per GPU, each part is
translated by its own process (no collectives), and the outputs are concatenated in order.

    python translate_distributed.py -model ckpt.pt -src input.txt -output pred.txt -gpus 0,1,2,3 [translate.py options]

Reference flow: translate_distributed.py:13-154 (split :116-138, ``Pool.map`` :143, concatenation :146-154).
"""
import multiprocessing as mp
import os
import shutil
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def split_file(path, n, tmpdir, tag):
    with open(path, encoding="utf-8") as fh:
        lines = fh.readlines()
    per = (len(lines) + n - 1) // n
    parts = []
    for i in range(n):
        p = os.path.join(tmpdir, "%s.%d" % (tag, i))
        with open(p, "w", encoding="utf-8") as out:
            out.writelines(lines[i * per:(i + 1) * per])
        parts.append(p)
    return parts


def run_part(args):
    argv, = args
    import translate
    translate.main(argv)
    return 0


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)

    def take(flag, default=None):
        if flag in argv:
            i = argv.index(flag)
            val = argv[i + 1]
            del argv[i:i + 2]
            return val
        return default

    gpus = [int(g) for g in str(take("-gpus", "0")).split(",") if g != ""]
    src, out, tgt = take("-src"), take("-output", "pred.txt"), take("-tgt")
    side_inputs = {flag: take(flag) for flag in ("-sub_src", "-past_src")}     # line-parallel to -src: split the same way
    take("-gpu")
    tmpdir = tempfile.mkdtemp(prefix="nmtg_translate_")
    try:
        src_parts = split_file(src, len(gpus), tmpdir, "src")
        tgt_parts = split_file(tgt, len(gpus), tmpdir, "tgt") if tgt else [None] * len(gpus)
        side_parts = {flag: split_file(path, len(gpus), tmpdir, flag.strip("-")) for flag, path in side_inputs.items() if path}
        out_parts = [os.path.join(tmpdir, "out.%d" % i) for i in range(len(gpus))]
        jobs = []
        for i, g in enumerate(gpus):
            a = argv + ["-src", src_parts[i], "-output", out_parts[i], "-gpu", str(g)]
            if tgt_parts[i]:
                a += ["-tgt", tgt_parts[i]]
            for flag, parts in side_parts.items():
                a += [flag, parts[i]]
            jobs.append((a,))
        with mp.get_context("spawn").Pool(len(gpus)) as pool:
            pool.map(run_part, jobs)
        with open(out, "w", encoding="utf-8") as fh:
            for p in out_parts:
                with open(p, encoding="utf-8") as part:
                    shutil.copyfileobj(part, fh)
    finally:
        shutil.rmtree(tmpdir, ignore_errors=True)


if __name__ == "__main__":
    main()
