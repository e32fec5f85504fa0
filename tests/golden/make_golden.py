"""Make the golden logits: the reference's own Qwen3ForCausalLM, run once on the
CPU in float32 on tiny random models.

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

The weights are this repository's seeded random weights (tests/helpers.py gives
the configurations and seeds), loaded into the reference model by their
checkpoint names; for the tied configuration the reference still wants an
``lm_head.weight`` key (mini_llm/checkpoint.py:340-343), so the embedding matrix
is passed under that name.  Outputs: ``tiny_<name>.json`` with the token ids and
the float32 logits ``[tokens, vocab]`` (rounded to 9 significant digits).
"""

import json
import random
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.dont_write_bytecode = True

from mini_llm.config import Qwen3Config  # noqa: E402  (the reference)
from mini_llm.model.qwen import Qwen3ForCausalLM  # noqa: E402

from llm_runtime_study_b200.config import architecture_for  # noqa: E402
from llm_runtime_study_b200.models.description import tensor_schema  # noqa: E402
from llm_runtime_study_b200.weights import random_state  # noqa: E402
from tests.helpers import TINY  # noqa: E402

LENGTHS = {"A": 19, "B": 33, "C": 21}


def main() -> None:
    for name, (raw, seed, _page) in TINY.items():
        arch = architecture_for(raw)
        schema = tensor_schema(arch.describe(arch.config_from_dict(raw)))
        state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
        reference_state = dict(state)
        reference_state.setdefault("lm_head.weight", state["model.embed_tokens.weight"])
        model = Qwen3ForCausalLM(Qwen3Config.from_dict(raw)).eval()
        model.load_state_dict(reference_state, strict=True)
        rng = random.Random(100 + seed)
        ids = [rng.randrange(raw["vocab_size"]) for _ in range(LENGTHS[name])]
        with torch.inference_mode():
            logits = model(torch.tensor([ids]))[0]
        payload = {"seed": seed, "token_ids": ids, "shape": list(logits.shape),
                   "logits": [float(f"{v:.9g}") for v in logits.reshape(-1).tolist()]}
        (HERE / f"tiny_{name}.json").write_text(json.dumps(payload))
        print(name, tuple(logits.shape), float(logits.abs().max()))


if __name__ == "__main__":
    main()
