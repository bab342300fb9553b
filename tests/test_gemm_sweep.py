"""GEMM shape sweep: CSV format and operand layouts (CPU), one small timed sweep (GPU)."""
import io

import pytest

from accera_b200 import gemm_sweep as gs

HEADER = "m,n,k,transA,transB,alpha,beta,lda,ldb,ldc\n"


def test_parse_full_rows():
    # the column order and the meaning of the flags are the reference benchmarker's
    # (tools/benchmarkers/gemm_opts.py:8-33)
    text = HEADER + "256,128,64,1,0,1,1,256,64,256\n\n# comment\n768,320,30522,0,1,1.0,0.5,768,30522,768\n"
    shapes = gs.parse_shapes(io.StringIO(text))
    assert len(shapes) == 2
    s0, s1 = shapes
    assert (s0.m, s0.n, s0.k, s0.transA, s0.transB, s0.alpha, s0.beta) == (256, 128, 64, True, False, 1.0, 1.0)
    assert (s0.lda, s0.ldb, s0.ldc) == (256, 64, 256)
    assert (s1.transA, s1.transB, s1.beta) == (False, True, 0.5)
    assert s1.flop == 2.0 * 768 * 320 * 30522


def test_parse_defaults_and_headerless():
    # defaults as in the reference's option record: alpha 1, beta 0, no transposition
    shapes = gs.parse_shapes(["m,n,k\n", "8,16,32\n"])
    assert shapes == [gs.GemmShape(8, 16, 32)]
    assert shapes[0].alpha == 1.0 and shapes[0].beta == 0.0 and not shapes[0].transA
    shapes = gs.parse_shapes(["8,16,32,0,1,2,0,8,32,8\n"])
    assert shapes[0].transB and shapes[0].alpha == 2.0
    # columns in another order
    shapes = gs.parse_shapes(["k,transB,n,m\n", "32,1,16,8\n"])
    assert (shapes[0].m, shapes[0].n, shapes[0].k, shapes[0].transB) == (8, 16, 32, True)
    assert gs.parse_shapes([]) == []


@pytest.mark.parametrize("text", [
    "m,n\n1,2\n",                       # k missing
    "m,n,k,bogus\n1,2,3,4\n",           # unknown column
    HEADER + "0,2,3,0,0,1,1,0,0,0\n",   # empty dimension
    HEADER + "1,2,3,7,0,1,1,0,0,0\n",   # flag that is not 0/1
    "m,n,k\n1,2,3,4\n",                 # more fields than columns
])
def test_parse_rejects(text):
    with pytest.raises(ValueError):
        gs.parse_shapes(io.StringIO(text))


def test_operand_strides():
    s = gs.GemmShape(100, 200, 300)
    assert gs.operand_strides(s) == ((300, 1), (200, 1), (200, 1))
    s = gs.GemmShape(100, 200, 300, transA=True, transB=True)
    assert gs.operand_strides(s) == ((1, 100), (1, 300), (200, 1))


def test_make_operands_layout_cpu():
    import torch
    for tA in (False, True):
        for tB in (False, True):
            s = gs.GemmShape(24, 40, 56, transA=tA, transB=tB)
            A, B, C = gs.make_operands(s, "h", torch.device("cpu"))
            sa, sb, sc = gs.operand_strides(s)
            assert tuple(A.shape) == (24, 56) and tuple(A.stride()) == sa
            assert tuple(B.shape) == (56, 40) and tuple(B.stride()) == sb
            assert tuple(C.shape) == (24, 40) and tuple(C.stride()) == sc
    A, B, C = gs.make_operands(gs.GemmShape(8, 8, 16), "i", torch.device("cpu"))
    assert A.dtype == torch.int8 and C.dtype == torch.int32
    A, B, C = gs.make_operands(gs.GemmShape(8, 8, 16), "u", torch.device("cpu"))
    assert A.dtype == torch.uint8 and int(A.max()) <= 8 and C.dtype == torch.int32
    A, B, C = gs.make_operands(gs.GemmShape(8, 8, 16), "h", torch.device("cpu"), out_letter="s")
    assert A.dtype == torch.float16 and C.dtype == torch.float32


def test_output_type_pairs():
    assert gs.output_type("h") == "h" and gs.output_type("h", "s") == "s" and gs.output_type("b", "s") == "s"
    assert gs.output_type("i") == "w" and gs.output_type("u", "w") == "w" and gs.output_type("s") == "s"
    for bad in (("i", "s"), ("h", "b"), ("s", "h")):
        with pytest.raises(ValueError):
            gs.output_type(*bad)


def test_write_results_roundtrip():
    recs = [dict(zip(gs.COLUMNS, gs.GemmShape(8, 16, 32, beta=1.0).as_row()), type="h", compute="auto",
                 batch_size=5, min_of_means_s=1e-5, mean_of_means_s=2e-5, tflops=0.8)]
    buf = io.StringIO()
    gs.write_results(recs, buf)
    lines = buf.getvalue().strip().splitlines()
    assert lines[0].startswith("m,n,k,transA,transB,alpha,beta,lda,ldb,ldc,type,compute")
    assert "torch_tflops" not in lines[0]
    # the result file is itself a valid shape file
    assert gs.parse_shapes([",".join(lines[0].split(",")[:10]), ",".join(lines[1].split(",")[:10])]) == \
        [gs.GemmShape(8, 16, 32, beta=1.0)]


def test_run_shape_needs_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        gs.run_shape(gs.GemmShape(8, 8, 16))


@pytest.mark.gpu
@pytest.mark.parametrize("type_letter,compute,tol", [
    ("h", "tensor_preferred", 2e-2), ("b", "tensor_preferred", 2e-2), ("s", "tensor_preferred", 2e-2),
    ("s", "simt", 1e-5), ("i", "auto", 0.0), ("u", "auto", 0.0), ("h>s", "tensor_preferred", 2e-2),
    ("b>s", "tensor_preferred", 2e-2)])
def test_sweep_small_gpu(type_letter, compute, tol, tmp_path):
    type_letter, _, out_letter = type_letter.partition(">")
    rows = ["256,256,256,0,0,1,1,256,256,256", "384,288,512,1,0,1,1,512,512,384", "384,288,512,0,1,1,0,384,288,384",
            "200,136,264,1,1,1,1,0,0,0"]
    if type_letter not in ("i", "u"):
        rows.append("128,64,96,0,1,0.5,2,0,0,0")
    shapes = gs.parse_shapes([HEADER] + [r + "\n" for r in rows])
    for s in shapes:
        rec = gs.run_shape(s, type_letter, compute, batches=2, batch_size=3, warmup=1, compare_torch=(type_letter == "h" and not out_letter),
                           out_letter=out_letter or None)
        assert rec["max_rel_err"] <= tol, rec
        assert rec["tflops"] > 0 and rec["min_of_means_s"] <= rec["mean_of_means_s"]
        if type_letter == "h" and not out_letter:
            assert rec["torch_tflops"] > 0


@pytest.mark.gpu
def test_sweep_cli_gpu(tmp_path):
    src = tmp_path / "shapes.csv"
    src.write_text(HEADER + "512,512,512,0,1,1,1,512,512,512\n1024,256,128,0,0,1,0,0,0,0\n")
    out = tmp_path / "res.csv"
    assert gs.main(["--input", str(src), "--type", "b", "--output", str(out), "--batches", "2", "--batch-size", "4"]) == 0
    lines = out.read_text().strip().splitlines()
    assert len(lines) == 3 and "tflops" in lines[0] and "max_rel_err" in lines[0]
