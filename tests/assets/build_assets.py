"""Regenerates the small offline test assets:

* ``tokenizer/``  -- a byte-level BPE tokenizer with a 2048-entry vocabulary (``tokenizer.json`` +
  ``tokenizer_config.json``) trained on the synthetic corpus below;
* ``c4_test/data.json`` -- 2000 JSON-lines documents with a ``text`` field (stand-in for the C4 test split);
* ``cc12m_test/cc12m-train-0000.tar`` -- 32 image-caption pairs in WebDataset layout (``<key>.jpg``, ``<key>.txt``,
  ``<key>.json``): drawn gradients and shapes of 256-400 pixels with captions that describe them (stand-in for a CC12M
  shard; the ``cc12m-test`` dataset of the FLUX and vision-language loaders).

The corpus is generated from a fixed word list with a seeded RNG, so the outputs are reproducible:
``python tests/assets/build_assets.py``.
"""

import json
import os
import random

HERE = os.path.dirname(os.path.abspath(__file__))
WORDS = (
    "the of and to in is that for it as was with be by on not he this are or his from at which but have an had they "
    "you were their one all we can her has there been if more when will would who so no out up into than them only "
    "time some could these two may then do first any my now such like our over man me even most made after also did "
    "many before must through years where much your way well down should because each just those people how too little "
    "state good very make world still own see men work long get here between both life being under never day same "
    "another know while last might us great old year off come since against go came right used take three small large "
    "number model train token layer tensor kernel memory data batch step loss grad weight shard rank device stream "
    "compute matrix vector attention expert router gate norm scale cache block table sum digit answer question what "
    "please solve add numbers result equals plus minus times total value answer"
).split()


def make_docs(n: int, seed: int) -> list[str]:
    rng = random.Random(seed)
    docs = []
    for _ in range(n):
        sents = []
        for _ in range(rng.randint(3, 40)):
            k = rng.randint(4, 18)
            words = [rng.choice(WORDS) for _ in range(k)]
            if rng.random() < 0.3:
                words.insert(rng.randrange(k), str(rng.randint(0, 99999)))
            s = " ".join(words)
            sents.append(s[0].upper() + s[1:] + rng.choice(".?!"))
        docs.append(" ".join(sents))
    return docs


def main() -> None:
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    docs = make_docs(2000, 1234)
    os.makedirs(os.path.join(HERE, "c4_test"), exist_ok=True)
    with open(os.path.join(HERE, "c4_test", "data.json"), "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    specials = ["<|begin_of_text|>", "<|end_of_text|>", "<|pad|>"]
    trainer = trainers.BpeTrainer(vocab_size=2048, special_tokens=specials,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    extra = ["[ANSWER] 12345", "Question: what is the sum of the digits 1 + 2 + 3 ?"] * 50
    tok.train_from_iterator(docs + extra, trainer)
    os.makedirs(os.path.join(HERE, "tokenizer"), exist_ok=True)
    tok.save(os.path.join(HERE, "tokenizer", "tokenizer.json"))
    with open(os.path.join(HERE, "tokenizer", "tokenizer_config.json"), "w") as f:
        json.dump({"bos_token": specials[0], "eos_token": specials[1], "pad_token": specials[2],
                   "add_bos_token": True, "add_eos_token": False, "model_max_length": 131072}, f, indent=1)


def write_custom_schedule() -> None:
    """``custom_schedule.csv``: one row per pipeline rank, actions ``<stage><F|B><micro-batch>``, for 2 ranks with 2 looped
    stages each and 8 micro-batches (what ``--parallelism.pipeline_parallel_schedule_csv`` reads): the interleaved 1F1B
    order spelled out action by action."""
    from torchtitan_b200.parallel.pp import build_actions, validate_actions

    rows = build_actions("Interleaved1F1B", 2, 4, 8, "loop")
    validate_actions(rows, 2, 4, 8, "loop")
    with open(os.path.join(HERE, "custom_schedule.csv"), "w") as f:
        for acts in rows:
            f.write(",".join(f"{a.stage}{a.kind}{a.mb}" for a in acts) + "\n")


def write_cc12m_test(n: int = 32, seed: int = 7) -> None:
    import io
    import tarfile

    from PIL import Image, ImageDraw

    rng = random.Random(seed)
    colours = {"red": (200, 40, 40), "green": (40, 160, 60), "blue": (40, 70, 200), "yellow": (220, 200, 50),
               "purple": (130, 60, 170), "orange": (230, 130, 40), "white": (235, 235, 235), "black": (25, 25, 25)}
    shapes = ("circle", "square", "triangle", "bar")
    os.makedirs(os.path.join(HERE, "cc12m_test"), exist_ok=True)
    with tarfile.open(os.path.join(HERE, "cc12m_test", "cc12m-train-0000.tar"), "w") as tar:
        for i in range(n):
            w, h = rng.randint(256, 400), rng.randint(256, 400)
            (bg_name, bg), (fg_name, fg) = rng.sample(sorted(colours.items()), 2)
            shape = rng.choice(shapes)
            img = Image.new("RGB", (w, h), bg)
            px = img.load()
            for y in range(h):                                   # vertical shading keeps the JPEG from being one flat block
                k = 0.75 + 0.25 * y / h
                for x in range(0, w):
                    px[x, y] = tuple(int(c * k) for c in bg)
            d = ImageDraw.Draw(img)
            cx, cy, r = rng.randint(w // 4, 3 * w // 4), rng.randint(h // 4, 3 * h // 4), rng.randint(30, min(w, h) // 4)
            if shape == "circle":
                d.ellipse((cx - r, cy - r, cx + r, cy + r), fill=fg)
            elif shape == "square":
                d.rectangle((cx - r, cy - r, cx + r, cy + r), fill=fg)
            elif shape == "triangle":
                d.polygon([(cx, cy - r), (cx - r, cy + r), (cx + r, cy + r)], fill=fg)
            else:
                d.rectangle((0, cy - r // 3, w, cy + r // 3), fill=fg)
            caption = f"a {fg_name} {shape} on a {bg_name} background"
            buf = io.BytesIO()
            img.save(buf, format="JPEG", quality=80)
            key = f"{i:09d}"
            meta = json.dumps({"key": key, "width": w, "height": h, "caption": caption}).encode()
            for name, data in ((f"{key}.jpg", buf.getvalue()), (f"{key}.json", meta), (f"{key}.txt", caption.encode())):
                info = tarfile.TarInfo(name)
                info.size = len(data)
                tar.addfile(info, io.BytesIO(data))


if __name__ == "__main__":
    main()
    write_custom_schedule()
    write_cc12m_test()
