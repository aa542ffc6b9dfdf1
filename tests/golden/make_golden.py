"""Extract known-answer vectors for the hot path from the reference's own files.

Run once in a checkout where the reference tree is available:

    python tests/golden/make_golden.py /path/to/reference

It reads (never executes) the haddock examples in
``src/Data/Array/Accelerate/{Language,Prelude}.hs`` and the regression tests
under ``src/Data/Array/Accelerate/Test/NoFib/{Issues,Misc}`` and writes
``tests/golden/reference_vectors.json``: for each case the expected result
(shape + flat values, or a list of tuples) together with the file and line it
was taken from.  The inputs and programs of the cases are restated in
``tests/test_oracle_golden.py`` next to the citation.
"""
import json
import os
import re
import sys

NUM = re.compile(r"-?\d+(?:\.\d+)?")


def parse_shape(text):
    m = re.search(r"\(Z((?:\s*:\.\s*\d+)+)\)", text)
    if m:
        return [int(x) for x in re.findall(r"\d+", m.group(1))]
    if re.search(r"Scalar Z", text) or re.search(r"fromList Z ", text):
        return []
    raise ValueError("no shape in: " + text[:80])


def doctest_output(lines, command, occurrence=1):
    """Output block that follows the `occurrence`-th haddock line `-- >>> command`."""
    seen = 0
    for i, l in enumerate(lines):
        if l.strip().startswith("-- >>>") and l.strip()[6:].strip() == command:
            seen += 1
            if seen == occurrence:
                out = []
                for m in lines[i + 1:]:
                    s = m.strip()
                    if s == "--" or s.startswith("-- >>>") or not s.startswith("--"):
                        break
                    out.append(s[2:])
                text = " ".join(out).strip()
                if text.startswith("("):
                    # a pair of arrays, as `filter` returns: "(Vector (Z :. 5) [..],Scalar Z [5])"
                    parts = []
                    for m in re.finditer(r"(Vector|Matrix|Array|Scalar)\s*(\(Z[^)]*\)|Z)\s*\[([^\]]*)\]", text):
                        sh = [int(x) for x in re.findall(r"\d+", m.group(2))]
                        parts.append({"shape": sh, "values": [int(v) for v in NUM.findall(m.group(3))]})
                    return i + 1, None, parts
                shape = parse_shape(text)
                body = text[text.index("["):]
                if "(" in body:
                    # tuples, shapes inside them written Z :. i :. j: keep the numbers of each tuple together
                    flat = body.replace("Z :.", "").replace(":.", ",")
                    tuples = re.findall(r"\(([^()]*)\)", flat)
                    return i + 1, shape, [[float(v) if "." in v else int(v) for v in NUM.findall(t)] for t in tuples]
                vals = [float(v) if "." in v else int(v) for v in NUM.findall(body)]
                if not vals and ("True" in body or "False" in body):
                    vals = [1 if w == "True" else 0 for w in re.findall(r"True|False", body)]
                return i + 1, shape, vals
    raise KeyError(command)


def issue_list(lines, name):
    """Values of `name = fromList (...) [ ... ]` in a regression test."""
    for i, l in enumerate(lines):
        if re.match(rf"{name}\s*=\s*fromList", l):
            text = l
            j = i
            while text.count("[") > text.count("]"):
                j += 1
                text += lines[j]
            shape = parse_shape(text)
            body = text[text.index("["):]
            tuples = re.findall(r"\(([^()]*)\)", body)
            if tuples:
                vals = [[float(v) if "." in v else int(v) for v in NUM.findall(t)] for t in tuples]
            else:
                vals = [float(v) if "." in v else int(v) for v in NUM.findall(body)]
            return i + 1, shape, vals
    raise KeyError(name)


def main(ref):
    base = os.path.join(ref, "src", "Data", "Array", "Accelerate")
    out = {}

    def add(key, path, line, shape, values):
        if shape is None:       # several arrays: one entry each, key_0, key_1
            for k, part in enumerate(values):
                out[f"{key}_{k}"] = {"source": f"{os.path.relpath(path, ref)}:{line}", "shape": part["shape"], "values": part["values"]}
            return
        out[key] = {"source": f"{os.path.relpath(path, ref)}:{line}", "shape": shape, "values": values}

    doc_cases = {
        "Language.hs": [
            ("generate_plus1", "run $ generate (I1 10) (\\(I1 i) -> i + 1) :: Vector Int", 1),
            ("map_plus1", "run $ map (+1) (use xs)", 1),
            ("zipWith_plus", "run $ zipWith (+) (use xs) (use ys)", 1),
            ("fold_plus_42", "run $ fold (+) 42 (use mat)", 1),
            ("maximum_segment_sum", "run $ maximumSegmentSum (use vec)", 1),
            ("scanl_vec", "run $ scanl (+) 10 (use vec)", 1),
            ("scanl_mat", "run $ scanl (+) 0 (use mat)", 1),
            ("scanl_prime_vec_res", "res", 1),
            ("scanl_prime_vec_sum", "sum", 1),
            ("scanl_prime_mat_res", "res", 2),
            ("scanl_prime_mat_sums", "sums", 1),
            ("scanl1_mat", "run $ scanl1 (+) (use mat)", 1),
            ("permute_histogram", "run $ histogram (use xs)", 1),
            ("permute_identity", "run $ identity 5 :: Matrix Int", 1),
            ("backpermute_transpose", "run $ backpermute (swap (shape mat')) swap mat'", 1),
            ("replicate_rows", "run $ replicate (constant (Z :. (4::Int) :. All)) (use vec)", 1),
            ("replicate_cols", "run $ replicate (lift (Z :. All :. (4::Int))) (use vec)", 1),
            ("replicate_two", "run $ replicate (constant (Z :. (2::Int) :. All :. (3::Int))) (use vec)", 1),
            ("replicate_rep0_unit", "run $ rep0 10 x", 1),
            ("replicate_rep0_vec", "run $ rep0 5 (use vec)", 1),
            ("replicate_rep1_vec", "run $ rep1 5 (use vec)", 1),
            ("generate_const", "run $ generate (I1 3) (\\_ -> 1.2) :: Vector Float", 1),
            ("fill_3", "run $ fill (constant (Z :. 3)) 1.2 :: Vector Float", 1),
            ("slice_row", "run $ slice (use mat) (constant (Z :. (2::Int) :. All))", 1),
            ("slice_point", "run $ slice (use mat) (constant (Z :. 4 :. 2 :: DIM2))", 1),
            ("slice_sl0_vec", "run $ sl0 (use vec) 4", 1),
            ("slice_sl0_mat", "run $ sl0 (use mat) 4", 1),
            ("slice_sl1_mat", "run $ sl1 (use mat) 4", 1),
            ("slice_sl1_cube", "run $ sl1 (use cube) 2", 1),
        ],
        "Prelude.hs": [
            ("foldSeg_mat", "run $ foldSeg (+) 0 (use mat) (use seg)", 1),
            ("sum_mat", "run $ sum (use mat)", 1),
            ("minimum_mat", "run $ minimum (use mat)", 1),
            ("maximum_mat", "run $ maximum (use mat)", 1),
            ("gather", "run $ gather (use from) (use input)", 1),
            ("scatter", "run $ scatter (use to) (fill (constant (Z:.10)) 0) (use input)", 1),
            ("scanlSeg_mat", "run $ scanlSeg (+) 0 (use mat) (use seg)", 1),
            ("scanl_primeSeg_res", "res", 1),
            ("scanl_primeSeg_sums", "sums", 1),
            ("scanl1Seg_mat", "run $ scanl1Seg (+) (use mat) (use seg)", 1),
            ("scanrSeg_mat", "run $ scanrSeg (+) 0 (use mat) (use seg)", 1),
            ("scanr_primeSeg_res", "res", 2),
            ("scanr_primeSeg_sums", "sums", 2),
            ("scanr1Seg_mat", "run $ scanr1Seg (+) (use mat) (use seg)", 1),
            ("indexed_vec", "run $ indexed (use xs)", 1),
            ("indexed_mat", "run $ indexed (use mat)", 1),
            ("zip_mats", "run $ zip (use m1) (use m2)", 1),
            ("foldAll_vec", "run $ foldAll (+) 42 (use vec)", 1),
            ("foldAll_mat", "run $ foldAll (+) 0 (use mat)", 1),
            ("all_even", "run $ all even (use mat)", 1),
            ("any_even", "run $ any even (use mat)", 1),
            ("product_mat", "run $ product (use mat)", 1),
            ("prescanl_vec", "run $ prescanl (+) 0 (use vec)", 1),
            ("postscanl_vec", "run $ postscanl (+) 42 (use vec)", 1),
            ("fill_10", "run $ fill (constant (Z:.10)) 0 :: Vector Float", 1),
            ("enumFromN_mat", "run $ enumFromN (constant (Z:.5:.10)) 0 :: Matrix Int", 1),
            ("enumFromStepN_mat", "run $ enumFromStepN (constant (Z:.5:.10)) 0 0.5 :: Matrix Float", 1),
            ("append_mats", "run $ use m1 ++ use m2", 1),
            ("concatOn_1", "run $ concatOn _1 (use m1) (use m2)", 1),
            ("concatOn_2", "run $ concatOn _2 (use m1) (use m2)", 1),
            ("filter_even_vec", "run $ filter even (use vec)", 1),
            ("filter_odd_mat", "run $ filter odd (use mat)", 1),
            ("gatherIf", "run $ gatherIf (use from) (use mask) (> 4) (use defaults) (use input)", 1),
            ("scatterIf", "run $ scatterIf (use to) (use mask) (> 4) (fill (constant (Z:.10)) 0) (use input)", 1),
            ("reverseOn_1", "run $ reverseOn _1 (use mat)", 1),
            ("reverseOn_2", "run $ reverseOn _2 (use mat)", 1),
            ("transposeOn_mat", "run $ transposeOn _1 _2 (use mat)", 1),
            ("transposeOn_box_12", "run $ transposeOn _1 _2 (use box)", 1),
            ("transposeOn_box_23", "run $ transposeOn _2 _3 (use box)", 1),
            ("transposeOn_box_13", "run $ transposeOn _1 _3 (use box)", 1),
            ("take_5", "run $ take 5 (use mat)", 1),
            ("drop_7", "run $ drop 7 (use mat)", 1),
            ("init_mat", "run $ init (use mat)", 1),
            ("tail_mat", "run $ tail (use mat)", 1),
            ("primes_100", "run $ primes 100", 1),
        ],
    }
    for fname, cases in doc_cases.items():
        path = os.path.join(base, fname)
        lines = open(path, encoding="utf-8").read().splitlines()
        for key, cmd, occ in cases:
            line, shape, vals = doctest_output(lines, cmd, occ)
            add(key, path, line, shape, vals)

    issues = os.path.join(base, "Test", "NoFib", "Issues")
    for fname, names in [("Issue137.hs", ["ref1"]), ("Issue185.hs", ["ref1", "ref2", "ref3", "ref4", "ref5", "ref6"]),
                         ("Issue228.hs", ["ref1"]), ("Issue362.hs", ["e1", "e2"]), ("Issue114.hs", ["ref1"])]:
        path = os.path.join(issues, fname)
        lines = open(path, encoding="utf-8").read().splitlines()
        for nm in names:
            line, shape, vals = issue_list(lines, nm)
            add(f"{fname[:-3].lower()}_{nm}", path, line, shape, vals)

    # Issue102: one expected array.  Issue119: eleven folds and segmented scans whose inputs, segment
    # descriptors and expected results are all literals of the test (every `fromList`, in file order,
    # under the name it is bound to, numbered per test).
    path = os.path.join(issues, "Issue102.hs")
    line, shape, vals = issue_list(open(path, encoding="utf-8").read().splitlines(), "ref1")
    add("issue102_ref1", path, line, shape, vals)
    path = os.path.join(issues, "Issue119.hs")
    big = {}
    current = None
    for i, l in enumerate(open(path, encoding="utf-8").read().splitlines()):
        m = re.match(r"(ref|test)(\d+)\s*=", l)
        if m:
            current = m.group(2)
        m = re.match(r"\s*(ref\d+|xs|seg|ps|rs)\s*=.*fromList\s*(\(Z[^)]*\)|Z)\s*\[([^\]]*)\]", l)
        if m and current:
            name = m.group(1) if not m.group(1).startswith("ref") else "ref"
            big[f"{current}_{name}"] = {"source": f"{os.path.relpath(path, ref)}:{i + 1}",
                                        "shape": [int(x) for x in re.findall(r"\d+", m.group(2))],
                                        "values": [int(v) for v in NUM.findall(m.group(3))]}
    dst119 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "issue119.json")
    json.dump(big, open(dst119, "w"), sort_keys=True)
    print(f"wrote {len(big)} arrays to {dst119}")

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    json.dump(out, open(dst, "w"), indent=1, sort_keys=True)
    print(f"wrote {len(out)} cases to {dst}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of AccelerateHS/accelerate>")
    main(sys.argv[1])
