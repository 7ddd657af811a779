"""Test infrastructure, not product code.

Writes patched copies of the few reference sources that hold the training
step's entry points, so that the reference library can be built once with its
step routed to libdlb200 the way INTEGRATION.md describes.  Nothing of the
reference is kept in this repository: the script finds each entry point in the
reference's checkout by its signature and inserts one hook line behind the
opening brace of its body; the copies go to a build directory.

    python dropin_patch.py <reference>/lib/deep-learning <out dir>

Patched: v1/learner/model.hpp (members that hold the library's context and model,
and the switch `set_b200`), and the definitions of forward_pass, compute_error,
backward_pass, update_derivatives, merge_mp_derivatives, update_weights_mp,
update_weights_st, get_loss, reset_loss.  The hooks are macros of
oracle/dropin_glue.h.
"""
import os
import re
import sys

# file -> [(regex that matches the start of the definition, hook line)]
HOOKS = {
    "v1/learner/fwp_st.cpp": [(r"^void Model::forward_pass\(", "DLB_DROPIN_FORWARD(batch_size, ptr_array_inputs_received)")],
    "v1/learner/compute_error.cpp": [(r"^void Model::compute_error\(", "DLB_DROPIN_ERROR(batch_size, Ym)")],
    "v1/learner/bwp_st.cpp": [(r"^void Model::backward_pass\(", "DLB_DROPIN_BACKWARD(batch_size)")],
    "v1/learner/update_derivative_fwp_st.cpp": [(r"^void Model::update_derivatives\(", "DLB_DROPIN_DERIVATIVES(batch_size)")],
    "v1/learner/merge.cpp": [(r"^void Model::merge_mp_derivatives\(", "DLB_DROPIN_MERGE()")],
    "v1/learner/model.cpp": [(r"^\s*void Model::update_weights_mp\(", "DLB_DROPIN_UPDATE(batch_size, training_size)"),
                             (r"^\s*void Model::update_weights_st\(", "DLB_DROPIN_UPDATE(batch_size, training_size)")],
    "v1/learner/loss.cpp": [(r"^double Model::get_loss\(ENV::TYPE", "DLB_DROPIN_GET_LOSS(env)"),
                            (r"^void Model::reset_loss\(", "DLB_DROPIN_RESET_LOSS()")],
}
MEMBERS = """  // --- drop-in (oracle/dropin_glue.cpp): the step runs in libdlb200 while b200_on ---
  void *b200_ctx = nullptr;
  void *b200_model = nullptr;
  bool b200_on = false;
  bool set_b200(bool on, int device);
"""


def insert_after_body_brace(lines, start, hook):
    """Inserts `hook` after the first '{' at or after line `start` that opens the
    function body (the parameter list has no braces)."""
    for i in range(start, min(start + 40, len(lines))):
        if "{" in lines[i]:
            indent = re.match(r"\s*", lines[i + 1]).group(0) if i + 1 < len(lines) else "  "
            lines.insert(i + 1, f"{indent}{hook}\n")
            return
    raise SystemExit(f"no body brace after line {start}")


def main(src_root, out_root):
    for rel, hooks in HOOKS.items():
        with open(os.path.join(src_root, rel)) as f:
            lines = f.readlines()
        for pattern, hook in hooks:
            hits = [i for i, l in enumerate(lines) if re.search(pattern, l)]
            if len(hits) != 1:
                raise SystemExit(f"{rel}: {len(hits)} matches for {pattern}")
            insert_after_body_brace(lines, hits[0], hook)
        # the hook macros
        last_include = max(i for i, l in enumerate(lines) if l.startswith("#include"))
        lines.insert(last_include + 1, '#include "dropin_glue.h"\n')
        dst = os.path.join(out_root, "deep-learning", rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        with open(dst, "w") as f:
            f.writelines(lines)
    rel = "v1/learner/model.hpp"
    with open(os.path.join(src_root, rel)) as f:
        lines = f.readlines()
    hits = [i for i, l in enumerate(lines) if re.match(r"^class Model \{", l)]
    if len(hits) != 1 or "public:" not in lines[hits[0] + 1]:
        raise SystemExit("model.hpp: class Model { public: not found")
    lines.insert(hits[0] + 2, MEMBERS)
    dst = os.path.join(out_root, "deep-learning", rel)
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    with open(dst, "w") as f:
        f.writelines(lines)
    print("patched", len(HOOKS) + 1, "files into", out_root)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
