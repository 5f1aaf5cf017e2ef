"""A C program builds against the shipped headers and links the host library through `bshmem-config`, the API
reference generator runs, and the CMake package file names both libraries."""
import subprocess
import sys
import textwrap
from pathlib import Path

from roc_shmem_b200 import _native, docs, pkgconfig


def test_c_consumer_builds_and_runs(tmp_path):
    _native.host_lib()                                   # make sure the library exists
    src = tmp_path / "app.c"
    src.write_text(textwrap.dedent("""
        #include <stdio.h>
        #include "bshmem.h"
        int main(void) {
          void* world = 0; bshmem_handle_t h = 0;
          if (bshmem_cpu_world_create(0, 1, 1 << 20, &world) != BSHMEM_OK) return 1;
          if (bshmem_cpu_init(world, 0, 0, &h) != BSHMEM_OK) return 2;
          long* x = (long*)bshmem_malloc(h, 8 * sizeof(long));
          long v = 42;
          if (!x || bshmem_ctx_putmem(h, BSHMEM_CTX_DEFAULT, x, &v, sizeof v, 0) != BSHMEM_OK || x[0] != 42) return 3;
          bshmem_free(h, x);
          bshmem_finalize(h);
          bshmem_cpu_world_destroy(world);
          puts("C_CONSUMER_OK");
          return 0;
        }"""))
    p = pkgconfig.paths()
    exe = tmp_path / "app"
    cmd = ["gcc", str(src), f"-I{p['includedir']}", f"-L{p['libdir']}", f"-Wl,-rpath,{p['libdir']}", "-lbshmem_host", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "C_CONSUMER_OK" in r.stdout, r.stdout + r.stderr


def test_api_reference_and_cmake_package(tmp_path):
    text = docs.generate()
    for name in ("bshmem_malloc", "bshmem_team_split_strided", "putmem_signal", "team_reduce", "ctx_atomic_fetch_add",
                 "bshmem_gpu_group_collective_noalloc"):
        assert name in text
    cm = (Path(pkgconfig.paths()["cmakedir"]) / "bshmemConfig.cmake").read_text()
    assert "bshmem::host" in cm and "bshmem::cuda" in cm
    out = subprocess.run([sys.executable, "-m", "roc_shmem_b200.pkgconfig", "--cflags", "--libs"], capture_output=True, text=True)
    assert "-lbshmem_host" in out.stdout and "csrc/include" in out.stdout


def test_loader_uses_an_existing_library_without_rebuilding(monkeypatch):
    """Every rank of a multi-rank job imports the package at the same time: an existing library must be loaded as it
    is (no compiler run at import, even when a source file is newer), a missing one is built once under the lock, and
    B200SHMEM_AUTO_REBUILD=1 brings the rebuild-at-import behaviour back for a developer."""
    from roc_shmem_b200 import build
    _native.host_lib()
    calls = []
    monkeypatch.setattr(build, "build_host", lambda *a, **k: calls.append("host"))
    monkeypatch.setattr(_native, "_libs", {})
    monkeypatch.delenv("B200SHMEM_AUTO_REBUILD", raising=False)
    assert _native.load("libbshmem_host.so") is not None and calls == []
    monkeypatch.setattr(_native, "_libs", {})
    monkeypatch.setenv("B200SHMEM_AUTO_REBUILD", "1")
    assert _native.load("libbshmem_host.so") is not None and calls == ["host"]
    with _native._build_lock():                              # the lock file lives next to the libraries
        assert (Path(_native._LIB_DIR) / ".build.lock").exists()


def test_porting_guide_targets_exist():
    """Every name the porting guide sends a ROC_SHMEM user to is declared in a public header or is an attribute of the
    Python classes, and the guide covers the reference header's untyped entry points."""
    import re

    import roc_shmem_b200 as shmem
    from roc_shmem_b200.runtime import Context, Runtime, Team
    assert docs.porting_targets_missing() == []
    classes = {"Runtime": Runtime, "Context": Context, "Team": Team}
    for ref, (_host, _dev, py, _note) in docs.PORTING.items():
        for cls, attr in re.findall(r"(Runtime|Context|Team)\.(\w+)", py):
            assert hasattr(classes[cls], attr) or attr in ("my_pe", "n_pes", "team"), (ref, cls, attr)
        for attr in re.findall(r"roc_shmem_b200\.(\w+)", py):
            assert hasattr(shmem, attr), (ref, attr)
    for must in ("init", "finalize", "malloc", "putmem", "getmem_nbi", "ctx_create", "wg_init", "wg_team_create_ctx",
                 "ctx_wg_team_sync", "team_split_strided", "barrier_all", "ptr", "timer", "global_exit"):
        assert must in docs.PORTING
    text = docs.porting_guide()
    assert "| `putmem` |" in text and "Typed families" in text


def test_cmake_build_install_and_consumer(tmp_path):
    """The repository's CMakeLists.txt builds the host library (BSHMEM_CUDA=OFF keeps the test short; the CUDA targets
    use the same file), installs headers + library + package files, and a consumer project finds the installed
    package with find_package(bshmem) and runs."""
    import shutil
    if shutil.which("cmake") is None:
        import pytest
        pytest.skip("cmake is not installed")
    root = Path(__file__).resolve().parents[1]
    build, prefix = tmp_path / "build", tmp_path / "prefix"
    for cmd in (["cmake", "-S", str(root), "-B", str(build), "-DBSHMEM_CUDA=OFF"],
                ["cmake", "--build", str(build), "-j", "8"],
                ["cmake", "--install", str(build), "--prefix", str(prefix)]):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert (prefix / "include" / "bshmem" / "bshmem.h").exists() and (prefix / "include" / "bshmem" / "bshmem_device.cuh").exists()
    app = tmp_path / "app"
    app.mkdir()
    (app / "CMakeLists.txt").write_text(textwrap.dedent("""
        cmake_minimum_required(VERSION 3.24)
        project(app LANGUAGES C CXX)
        find_package(bshmem REQUIRED)
        add_executable(app app.c)
        target_link_libraries(app PRIVATE bshmem::bshmem_host)
        """))
    (app / "app.c").write_text(textwrap.dedent("""
        #include <stdio.h>
        #include "bshmem.h"
        int main(void) {
          void* world = 0; bshmem_handle_t h = 0;
          if (bshmem_cpu_world_create(0, 1, 1 << 20, &world) != BSHMEM_OK) return 1;
          if (bshmem_cpu_init(world, 0, 0, &h) != BSHMEM_OK) return 2;
          int* x = (int*)bshmem_malloc(h, 4 * sizeof(int));
          int r = -1;
          x[0] = 5;
          if (bshmem_team_reduce_root(h, BSHMEM_TEAM_WORLD, BSHMEM_INT32, BSHMEM_SUM, &x[1], &x[0], 1, 0) != BSHMEM_OK) return 3;
          r = x[1];
          bshmem_free(h, x);
          bshmem_finalize(h);
          bshmem_cpu_world_destroy(world);
          printf("CMAKE_CONSUMER_OK %d\\n", r);
          return r == 5 ? 0 : 4;
        }"""))
    r = subprocess.run(["cmake", "-S", str(app), "-B", str(app / "b"), f"-DCMAKE_PREFIX_PATH={prefix}"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run(["cmake", "--build", str(app / "b")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run([str(app / "b" / "app")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "CMAKE_CONSUMER_OK 5" in r.stdout, r.stdout + r.stderr
