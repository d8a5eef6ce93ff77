"""CPU test: a translation unit written against Sapphire's own leaf signatures
compiles with the compat header and links against the library (nothing is run:
there is no GPU here)."""
import os
import subprocess
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SNIPPET = textwrap.dedent('''
    #include "sapphire_b200_compat.hpp"
    // what Sources/Sapphire/compute/BasicOps.cpp:232-247 hands to BroadcastWith2Inputs
    using LeafFn = void (*)(unsigned int, float*, const float*, const float*, unsigned int,
                            unsigned int, unsigned int, int);
    int main(int argc, char**)
    {
        LeafFn leaf = Sapphire::Compute::Dense::Cuda::Gemm;
        auto bc = Sapphire::Compute::Dense::Cuda::GemmMatrixWiseBroadcast;
        auto sp = Sapphire::Compute::Sparse::Cuda::Gemm;
        static_assert(sizeof(SparseMatrix) == 48, "Sapphire's SparseMatrix is 48 bytes");
        if (argc > 100) {             // never true: the calls only have to link
            leaf(0, nullptr, nullptr, nullptr, 1, 1, 1, 0);
            bc(nullptr, nullptr, nullptr, 1, 1, 1, 1, false, false, 0);
            sp(nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, false);
        }
        auto plan = sb200::compat::PlanGemm({4, 8, 8}, {4, 8, 8}, {4, 8, 8});
        return plan.size() == 1 ? 0 : 1;
    }
''')


def test_sapphire_signature_shims_compile_and_link(tmp_path):
    src = tmp_path / "leaf_user.cpp"
    src.write_text(SNIPPET)
    exe = tmp_path / "leaf_user"
    lib_dir = os.path.join(ROOT, "sapphire_b200")
    cmd = ["g++", "-std=c++17", "-I", os.path.join(lib_dir, "compat"), str(src), "-o", str(exe),
           "-L", lib_dir, "-l:libsapphire_b200.so", f"-Wl,-rpath,{lib_dir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    # the host-only planner runs without a GPU
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
