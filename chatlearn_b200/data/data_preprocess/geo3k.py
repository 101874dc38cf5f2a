"""Geometry3K (vision) → prompt records (chatlearn/data/data_preprocess/geo3k.py).  The
images stay in the record (``images``); the vision prompt pipeline turns them into pixels."""
from .common import record, run_converter

DATA_SOURCE = "hiyouga/geometry3k"
INSTRUCTION = (r"You FIRST think about the reasoning process as an internal monologue and then provide the final answer. "
               r"The reasoning process MUST BE enclosed within <think> </think> tags. "
               r"The final answer MUST BE put in \boxed{}.")


def messages(problem: str, n_images: int):
    content = [{"type": "image"} for _ in range(n_images)] + [{"type": "text", "text": problem.replace("<image>", "") + " " + INSTRUCTION}]
    return [{"role": "user", "content": content}]


def convert(ex, split, idx, agent=False):
    imgs = ex.get("images") or []
    r = record(DATA_SOURCE, messages(ex["problem"], len(imgs)), ex["answer"], split, idx, ability="math",
               extra={"question": ex["problem"]},
               agent_name="geo3k_agent" if agent else None,
               agent_cfg_path="template/agent/geo3k_eval.yaml" if agent else None)
    r["images"] = [im.get("path") or im.get("bytes") if isinstance(im, dict) else im for im in imgs]
    r["images"] = [x.hex() if isinstance(x, (bytes, bytearray)) else x for x in r["images"]]
    return r


if __name__ == "__main__":
    run_converter(__doc__, "~/data/geo3k", convert)
