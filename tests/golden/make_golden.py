"""Writes tests/golden/tiny_{A,B}.{json,f32}: logits of the C++ twin
(tests/twin/qwen3_twin.cpp) at a few positions of one prompt, on the tiny
configurations A and B with random weights of a fixed seed.

They rest on the reference's formulas, not on its output: bigmah/llmoxide is
Rust over GGUF and can be neither compiled nor imported where this runs.

    python tests/golden/make_golden.py
"""

import json
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

from tiny_configs import ALL, make_folder, prompts  # noqa: E402
from twin_util import twin_logits  # noqa: E402

SEED = 1234
POSITIONS = [0, 1, 12, 24]

if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as tmp:
        for name in ("A", "B"):
            vocab = ALL[name]["vocab_size"]
            toks = prompts(vocab, [25], seed=77)[0]
            folder = make_folder(tmp, name, "float32", seed=SEED)
            logits = twin_logits(folder, toks, 13, vocab)[POSITIONS]
            logits.astype("<f4").tofile(HERE / f"tiny_{name}.f32")
            (HERE / f"tiny_{name}.json").write_text(json.dumps(
                dict(config=name, seed=SEED, tokens=toks, positions=POSITIONS, vocab=vocab,
                     made_by="tests/twin/qwen3_twin.cpp, prefix of 13 tokens then one by one")) + "\n")
            print(f"tiny_{name}: {logits.shape}")
