"""TEST INFRASTRUCTURE ONLY.  Cuts the named CUDA functions out of the mounted reference tree
so that they can be compiled, unmodified, behind oracle/ref_stage_wrapper.cu.

    python extract_reference_kernels.py <reference root> <output file>

The output is a build intermediate: the Makefile writes it to a temporary directory and only
the compiled library lands in oracle/_ref/.  A function is located by its definition line
(`__global__ void NAME(` or `__device__ TYPE NAME(`) and copied up to the brace that closes its
body, so the recipe follows the source if lines move."""
import re
import sys

WANTED = {
    # reference file (path inside its tree) -> functions, in an order that compiles
    "src/nvfp4_cutlass.cu": [
        "gelu", "reduce_expert_routes", "initialize_route_indices", "sorted_lower_bound",
        "quantize_bf16_sorted_moe", "configure_dynamic_grouped",
        "sort_and_configure_dynamic_grouped", "count_sort_and_configure_dynamic_grouped",
        "block_sort_and_configure_dynamic_grouped", "geglu_quantize_sorted_moe",
    ],
    "src/cuda/kernels/routing_sampling.cuh": ["route_128_top8_kernel"],
}


def cut(text, name):
    pattern = re.compile(r"^(?:__global__|__device__)[^\n;{]*\b" + re.escape(name) + r"\s*\(", re.M)
    match = pattern.search(text)
    if not match:
        raise SystemExit(f"function {name} not found")
    start = match.start()
    open_brace = text.index("{", match.end())
    # the signature must not contain a body of its own (default arguments have no braces)
    depth, i = 0, open_brace
    while True:
        c = text[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                break
        i += 1
    return text[start:i + 1]


def main():
    root, out = sys.argv[1], sys.argv[2]
    parts = []
    for path, names in WANTED.items():
        with open(f"{root}/{path}") as f:
            text = f.read()
        for name in names:
            parts.append(f"// ---- {path}: {name}\n" + cut(text, name) + "\n")
    with open(out, "w") as f:
        f.write("\n".join(parts))


if __name__ == "__main__":
    main()
