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
