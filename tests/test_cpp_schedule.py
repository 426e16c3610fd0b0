"""A user schedule written against the reference's Rewriter signatures (tests/cpp/api_schedule_recipe.cc:
the SGEMM recipe of the reference's MatmulOptimizer, src/Optimizer/Optimizer.cc:383-548) runs on
the own IR, and every stage has the structure the reference documents in README.md:189-1607
(problem 4096 x 2048 x 1024, tiles 128 x 128 x 8, 8 x 8 per thread, float4 accesses).

Index expressions are compared by value, not by spelling: the printed expressions are evaluated
for sample thread / block / loop indices and held to the formulas the README stages show (MLIR
prints them simplified, e.g. `%arg2 * 8 + %arg3 floordiv 2` for `(%arg2 * 16 + %arg3) floordiv 2`).
"""
import itertools
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def stages(tmp_path_factory):
    from kernelcodegen_b200 import build

    exe = tmp_path_factory.mktemp("cpp") / "api_schedule_recipe"
    build.compile_program(ROOT / "tests" / "cpp" / "api_schedule_recipe.cc", exe)
    res = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    sections, name = {}, None
    for line in res.stdout.splitlines():
        if line.startswith("=== "):
            name = line[4:].strip()
            sections[name] = []
        elif name:
            sections[name].append(line)
    return {k: "\n".join(v) for k, v in sections.items()}


def loops(text):
    return [(int(a), int(b), int(c or 1)) for a, b, c in
            re.findall(r"affine\.for %\w+ = (\d+) to (\d+)(?: step (\d+))?", text)]


def accesses(text, kind, memref):
    """[(index texts..., width)] of every `kind` (vector_load / vector_store / load / store) on `memref`."""
    out = []
    pat = rf"affine\.{kind} (?:%\w+, )?{re.escape(memref)}\[(.*)\] : memref<[^>]*>(?:, vector<(\d+)xf32>)?"
    for m in re.finditer(pat, text):
        depth, cur, parts = 0, "", []
        for ch in m.group(1):
            if ch == "," and depth == 0:
                parts.append(cur.strip())
                cur = ""
                continue
            depth += ch in "(["
            depth -= ch in ")]"
            cur += ch
        parts.append(cur.strip())
        out.append((parts, int(m.group(2) or 1)))
    return out


def evaluate(expr, env):
    """Value of a printed index expression; %names come from `env`, %cN constants from their name."""
    py = expr.replace(" floordiv ", " // ").replace(" mod ", " % ")
    py = re.sub(r"%c(\d+)(?:_\d+)?\b", r"\1", py)
    py = re.sub(r"%(\w+)", lambda m: str(env[m.group(1)]), py)
    return eval(py, {"__builtins__": {}})  # arithmetic only


def names_in(expr):
    return sorted(set(re.findall(r"%(arg\d+)", expr)), key=lambda s: int(s[3:]))


# In every stage: %arg3, %arg4 = blockIdx (y, x); %arg5, %arg6 = threadIdx (y, x) (function arguments are %arg0..2).
BY, BX, TY, TX = "arg3", "arg4", "arg5", "arg6"
SAMPLES = [(0, 0, 0, 0), (3, 7, 1, 2), (15, 15, 31, 15), (8, 1, 5, 9), (2, 13, 30, 0)]   # (ty, tx, by, bx)


def check(expr, formula, extra_names):
    """expr == formula(ty, tx, by, bx, *extras) on the samples; the names of expr other than the four
    parallel indices are bound, in order of appearance by number, to `extra_names`' sample values."""
    others = [n for n in names_in(expr) if n not in (BY, BX, TY, TX)]
    assert len(others) <= len(extra_names), (expr, others)
    for ty, tx, by, bx in SAMPLES:
        for extras in itertools.product(*[extra_names[i] for i in range(len(extra_names))]):
            env = {TY: ty, TX: tx, BY: by, BX: bx}
            env.update({n: extras[i] for i, n in enumerate(others)})
            assert evaluate(expr, env) == formula(ty, tx, by, bx, *extras), (expr, env)


def test_alloc_buffer_stage(stages):
    # README.md:232-279
    t = stages["alloc_buffer"]
    assert re.findall(r"memref\.alloc\(\) : (memref<[^>]*>)", t)[:7] == [
        "memref<8x128xf32, 2>", "memref<8x128xf32, 2>", "memref<4xf32, 3>", "memref<4xf32, 3>", "memref<8xf32, 3>",
        "memref<8xf32, 3>", "memref<8x8xf32, 3>"]


def test_read_stage(stages):
    # README.md:281-336: two copy loops `0 to 1` at the start of the k loop, float4 loads of A and B
    t = stages["read"]
    assert loops(t)[2:5] == [(0, 1024, 8), (0, 1, 1), (0, 1, 1)]
    (a_idx, wa), = accesses(t, "vector_load", "%arg0")
    (b_idx, wb), = accesses(t, "vector_load", "%arg1")
    assert wa == wb == 4
    ks, ivs = (0, 8, 1016), (0,)
    # README.md:306: %0[%arg2 * 8 + %arg3 floordiv 2 + %arg5 * 128 + %arg0 * 128, (%arg3 mod 2) * 4 + %arg4]
    check(a_idx[0], lambda ty, tx, by, bx, iv: ty * 8 + tx // 2 + iv * 128 + by * 128, [ivs])
    check(a_idx[1], lambda ty, tx, by, bx, k, iv: (tx % 2) * 4 + k, [ks, ivs])
    # README.md:310: %1[(%arg2 * 16 + %arg3) floordiv 32 + %arg5 * 8 + %arg4, ((%arg2 * 16 + %arg3) mod 32) * 4 + %arg1 * 128]
    check(b_idx[0], lambda ty, tx, by, bx, k, iv: (ty * 16 + tx) // 32 + iv * 8 + k, [ks, ivs])
    check(b_idx[1], lambda ty, tx, by, bx, iv: ((ty * 16 + tx) % 32) * 4 + bx * 128, [ivs])
    assert len(accesses(t, "vector_store", "%4")) == 1 and len(accesses(t, "vector_store", "%5")) == 1


def test_write_stage(stages):
    # README.md:338-405: A goes to shared memory transposed, element by element; B as float4 rows
    t = stages["write"]
    (a_idx, wa), = accesses(t, "vector_store", "%0")
    (b_idx, wb), = accesses(t, "vector_store", "%1")
    assert (wa, wb) == (1, 4)
    check(a_idx[0], lambda ty, tx, by, bx, iv, e: (tx % 2) * 4 + e, [(0,), (0, 1, 2, 3)])
    check(a_idx[1], lambda ty, tx, by, bx, iv: ty * 8 + tx // 2 + iv * 128, [(0,)])
    check(b_idx[0], lambda ty, tx, by, bx, iv: (ty * 16 + tx) // 32 + iv * 8, [(0,)])
    check(b_idx[1], lambda ty, tx, by, bx, iv: ((ty * 16 + tx) % 32) * 4, [(0,)])
    assert t.count("gpu.barrier") == 2
    assert (0, 4, 1) in loops(t)          # the element loop of the transposed store


def test_read_frag_stage(stages):
    # README.md:407-482: two `0 to 2` loops at the start of the inner k loop fill the 8-float fragments
    t = stages["read_frag"]
    (a_idx, wa), = accesses(t, "vector_load", "%0")
    (b_idx, wb), = accesses(t, "vector_load", "%1")
    assert wa == wb == 4
    tid = lambda ty, tx: ty * 16 + tx
    check(a_idx[0], lambda ty, tx, by, bx, k: k, [(0, 3, 7)])
    check(a_idx[1], lambda ty, tx, by, bx, iv: ((tid(ty, tx) % 32) // 4 + ((tid(ty, tx) // 32) // 4 + iv * 2) * 8) * 4, [(0, 1)])
    check(b_idx[1], lambda ty, tx, by, bx, iv: (tx % 4 + ((tid(ty, tx) // 32) % 4 + iv * 4) * 4) * 4, [(0, 1)])
    assert loops(t).count((0, 2, 1)) == 2


def test_cache_read_stage(stages):
    # README.md:484-559: the product reads the fragments, not global memory
    t = stages["cache_read"]
    assert re.search(r"affine\.load %6\[%arg\d+\] : memref<8xf32, 3>", t)
    assert re.search(r"affine\.load %7\[%arg\d+\] : memref<8xf32, 3>", t)
    assert not accesses(t, "load", "%arg0") and not accesses(t, "load", "%arg1")


def test_cache_write_stage_covers_the_tile_once(stages):
    # README.md:561-640 (structure) with the thread layout of src/Optimizer/Optimizer.cc:365-377: every
    # element of a block's 128 x 128 tile of C is stored by exactly one (thread, i0, j0, i1, j1)
    t = stages["cache_write"]
    assert loops(t)[-4:] == [(0, 8, 4), (0, 8, 4), (0, 4, 1), (0, 4, 1)]
    (idx, w), = accesses(t, "store", "%arg2")
    others = [n for n in sorted(set(names_in(idx[0]) + names_in(idx[1])), key=lambda s: int(s[3:])) if n not in (BY, BX, TY, TX)]
    assert len(others) == 4                      # i0, j0, i1, j1 in loop order
    seen = set()
    for ty in range(16):
        for tx in range(16):
            for i0, j0 in itertools.product((0, 4), repeat=2):
                for i1, j1 in itertools.product(range(4), repeat=2):
                    env = {TY: ty, TX: tx, BY: 2, BX: 5, **dict(zip(others, (i0, j0, i1, j1)))}
                    seen.add((evaluate(idx[0], env) - 2 * 128, evaluate(idx[1], env) - 5 * 128))
    assert seen == set(itertools.product(range(128), repeat=2))


def test_vectorize_stage(stages):
    # README.md:723-802: the innermost store loop becomes `0 to 4 step 4` over float4 accesses
    t = stages["vectorize"]
    assert loops(t)[-1] == (0, 4, 4)
    assert accesses(t, "vector_load", "%8")[0][1] == 4 and accesses(t, "vector_store", "%arg2")[0][1] == 4


def test_pipeline_stage(stages):
    # README.md:804-921
    t = stages["pipeline"]
    types = re.findall(r"memref\.alloc\(\) : (memref<[^>]*>)", t)
    assert types.count("memref<2x8x128xf32, 2>") == 2 and types.count("memref<2x8xf32, 3>") == 2
    assert "memref<8x128xf32, 2>" not in types and "memref<8xf32, 3>" not in types
    # prefetch guards: iv + 2 * step <= ub
    assert t.count("+ 1008 >= 0") == 2 and t.count("+ 6 >= 0") == 2
    # halves: stores one iteration ahead, loads from the current one; copies in front of the loops use half 0
    assert len(re.findall(r"vector_store %\d+, %[01]\[\(%arg\d+ floordiv 8 \+ 1\) mod 2,", t)) == 2
    assert len(re.findall(r"vector_store %\d+, %[01]\[0,", t)) == 2
    assert len(re.findall(r"vector_load %[01]\[\(%arg\d+ floordiv 8\) mod 2, %arg\d+ \+ 1,", t)) == 2
    assert len(re.findall(r"affine\.load %[67]\[%arg\d+ mod 2, %arg\d+\]", t)) == 2
    # the global loads inside the loop read the next k slab
    assert re.search(r"vector_load %arg0\[.*\+ %arg\d+ \+ 8\]", t) and re.search(r"vector_load %arg1\[.* \+ %arg\d+ \+ 8,", t)


def test_detach_last_loop_stage(stages):
    # README.md:923-1063: the inner k loop runs 0 to 7; iteration 7 follows it with a constant index
    t = stages["detach_last_loop"]
    assert (0, 7, 1) in loops(t) and (0, 8, 1) in loops(t)
    assert re.search(r"%c7(_\d+)? = arith\.constant 7 : index", t)
    assert len(re.findall(r"affine\.load %[67]\[%c7(?:_\d+)? mod 2,", t)) == 2


def test_schedule_stage_orders_the_main_loop(stages):
    # README.md:1065-1351: global loads of the next slab, the k loop, the stores to shared memory and the
    # barrier, the last product, then the first fragments of the next slab
    t = stages["schedule"]
    body = t[t.index("= 0 to 1024 step 8"):]
    guard1 = body.index("+ 1008 >= 0")
    k_loop = body.index("= 0 to 7 {")
    guard2 = body.index("+ 1008 >= 0", guard1 + 1)
    barrier = body.index("gpu.barrier")
    last = body.index(">= 0)>(%c7")              # the fragment prefetch of the detached iteration: never true
    assert guard1 < k_loop < guard2 < barrier < last
    assert "vector_load %arg0[" in body[guard1:k_loop] and "vector_load %arg1[" in body[guard1:k_loop]
    assert "vector_load" not in body[guard2:barrier].replace("vector_load %4[", "").replace("vector_load %5[", "")
    assert t.count("gpu.barrier") == 2


def test_if_folding(stages):
    # the fragment prefetch guard (iv <= 6 inside a 0..7 loop) always holds and disappears; the slab guard stays
    t = stages["fold_if"]
    assert "+ 6 >= 0" not in t and t.count("+ 1008 >= 0") == 2
    assert ">= 0)>(%c7" not in t                 # the guards that can never hold are gone with their bodies


def test_unroll_and_unroll_attribute(stages):
    # README.md:1353-1607: loops of fewer than 4 iterations are unrolled; short ones left carry the attribute
    t = stages["unroll"]
    assert (0, 1, 1) not in loops(t) and (0, 2, 1) not in loops(t)
    u = stages["unroll_attribute"]
    marked = re.findall(r'\} attributes \{affine\.loop = "unroll"', u)
    assert len(marked) >= 10
    assert '= 0 to 1024 step 8 {' in u
    tail = u[u.index("= 0 to 1024 step 8 {"):]
    k_end = re.search(r"\n        \}( attributes \{[^}]*\})?\n", tail)
    assert k_end and "unroll" not in (k_end.group(1) or "")     # 128 iterations: not marked
