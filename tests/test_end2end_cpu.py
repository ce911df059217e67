"""The end-to-end aggregator (reference: A100-evaluation/EndToEnd/build_run.py): CSV reading, the derived-time
formula and the print format, on a hand-made table; the core-conv counts of TK-ResNet-18 read off the model."""
import torch

from tdc_b200 import end2end


def test_derived_time_and_report(tmp_path):
    p = tmp_path / "layers.csv"
    p.write_text("N,C,H,W,FFT,WINO,GEMM,TVM,TDC,a,b,c,d,diff\n"
                 "32,64,56,56,0.5,nan,0.10,0.08,0.04,1,1,2.5,2,0\n"
                 "32,32,56,56,0.4,0.3,0.06,0.05,0.03,1,1,2,1.6,0\n")
    layers = end2end.read_layer_csv(str(p))
    assert set(layers) == {(64, 32, 56, 56), (32, 32, 56, 56)} and layers[(64, 32, 56, 56)]["tdc"] == 0.04
    counts = {(64, 32, 56, 56): 1, (32, 32, 56, 56): 3}
    # 2.0 - (1*(0.10-0.04) + 3*(0.06-0.03)) = 1.85 ; against the TVM column: 2.0 - (0.02 + 3*0.01)
    assert abs(end2end.derived_time(2.0, counts, layers) - 1.85) < 1e-12
    assert abs(end2end.derived_time(2.0, counts, layers, ours="tvm") - 1.95) < 1e-12
    out = end2end.report("resnet18-tk", {"resnet18-tk": 2.0, "resnet18-tk-derived": 1.85})
    assert out == "resnet18-tk(Run time),resnet18-tk-derived(Run time)\n2.0(ms),1.85(ms)"


def test_core_conv_counts_of_tk_resnet18(built):
    import tdc_b200 as T
    m = T.tkc_resnet18()
    c = end2end.core_conv_counts(m, torch.zeros(1, 3, 224, 224))
    assert sum(c.values()) == 16
    assert c[(32, 32, 56, 56)] == 4 and c[(32, 64, 56, 56)] == 1 and c[(64, 64, 28, 28)] == 3 and c[(256, 256, 7, 7)] == 3
    v = end2end.core_conv_counts(T.tkc_vgg16(), torch.zeros(1, 3, 224, 224))
    assert sum(v.values()) == 12 and v[(32, 32, 224, 224)] == 1 and v[(256, 256, 14, 14)] == 3


def test_reference_row_of_the_layer_driver_is_read_back(built, tmp_path):
    """`layer_driver --reference-row` writes the reference's row (N,C,H,W,FFT,WINO,GEMM,TVM,TDC,ratios,diff) with nan
    for what was not measured; the aggregator reads it like the reference's own CSVs."""
    from tdc_b200 import end2end
    p = tmp_path / "B200-layers-eval.csv"
    p.write_text("64,64,56,56,0.115488,nan,0.046656,nan,0.036976,3.123323,nan,1.261791,nan,0\n"
                 "512,512,7,7,0.350688,nan,0.702912,nan,0.046000,7.623652,nan,15.280696,nan,0\n")
    rows = end2end.read_layer_csv(str(p))
    assert rows[(64, 64, 56, 56)]["gemm"] == 0.046656 and rows[(512, 512, 7, 7)]["tdc"] == 0.046
    assert rows[(64, 64, 56, 56)]["wino"] != rows[(64, 64, 56, 56)]["wino"]          # nan
    assert abs(end2end.derived_time(2.0, {(64, 64, 56, 56): 2, (512, 512, 7, 7): 1}, rows)
               - (2.0 - 2 * (0.046656 - 0.036976) - (0.702912 - 0.046))) < 1e-12


def test_cudnn_baseline_tool_is_built_where_cudnn_headers_exist(built):
    import os
    import tdc_b200
    have_headers = any(os.path.exists(os.path.join(d, "cudnn.h")) for d in
                       ("/usr/include/x86_64-linux-gnu", "/usr/include", "/usr/local/cuda/include"))
    exe = os.path.join(os.path.dirname(tdc_b200.__file__), "cudnn_layer_baseline")
    assert os.path.exists(exe) == have_headers
