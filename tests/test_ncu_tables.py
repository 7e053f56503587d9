"""The ncu CSV totals (kernel count, summed latency, DRAM MB read) against hand-made exports in both CSV shapes."""
import pytest

from souffle_models_b200 import ncu_tables

WIDE = '''"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","gpu__time_duration.sum","dram__bytes_read.sum"
"","","","","","","","","","","","usecond","Mbyte"
"0","1","python","h","void souffle_megakernel<0>(CallArgs)","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","2,100.5","450.25"
"1","1","python","h","transpose_kn_to_nk(const __half *, __half *, int, int)","1","7","(32, 8, 1)","(24, 24, 1)","0","10.0","5.5","N/A"
"2","1","python","h","void souffle_megakernel<0>(CallArgs)","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","2,099.5","nan"
'''

LONG = '''==PROF== Connected to process 1
"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"
"0","1","python","h","void souffle_megakernel<0>(CallArgs)","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","2100500"
"0","1","python","h","void souffle_megakernel<0>(CallArgs)","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","byte","472121344"
"1","1","python","h","souffle_lstm_wavefront(LstmParams)","1","7","(512, 1, 1)","(80, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","427.0"
"1","1","python","h","souffle_lstm_wavefront(LstmParams)","1","7","(512, 1, 1)","(80, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Kbyte","10,240"
'''


def test_wide_export(tmp_path):
    p = tmp_path / "wide.csv"
    p.write_text(WIDE)
    t = ncu_tables.totals(str(p))
    assert t["kernels"] == 3
    assert t["latency_ms"] == pytest.approx((2100.5 + 5.5 + 2099.5) / 1000.0)
    assert t["dram_read_mb"] == pytest.approx(450.25)          # N/A and nan count as zero
    only = ncu_tables.totals(str(p), r"souffle_megakernel")
    assert only["kernels"] == 2 and only["latency_ms"] == pytest.approx(4.2)


def test_long_export(tmp_path):
    p = tmp_path / "long.csv"
    p.write_text(LONG)
    t = ncu_tables.totals(str(p))
    assert t["kernels"] == 2
    assert t["latency_ms"] == pytest.approx(2.1005 + 0.427)
    assert t["dram_read_mb"] == pytest.approx(472121344 / 2**20 + 10.0)


def test_missing_header(tmp_path):
    p = tmp_path / "bad.csv"
    p.write_text("nothing,here\n")
    with pytest.raises(ValueError):
        ncu_tables.read_launches(str(p))


def test_profile_cases_lists_every_model_and_refuses_unknown_names():
    import pytest
    from souffle_models_b200 import profile_cases
    for name in ("bert_layer", "bert_base", "bert_layer_s384", "bert_layer_s384_plan", "lstm", "swin_mlp", "swin_pair", "swin_stage",
                 "se_module"):
        assert name in profile_cases.__doc__
    assert len(profile_cases.SE_SHAPES) == 10
    with pytest.raises(SystemExit):
        profile_cases.make_case("no_such_case")
