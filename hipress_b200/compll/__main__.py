"""Command line of the generator, flags as in the reference's GCGen.py
(src/CompLL/GCGen/GCGen.py:5-11 of mark14wu/hipress): ``input_file -b -w -r -f``.
The reference parses ``-f`` and ignores it (always MXNet); here ``-f torch`` is the
one supported target and anything else is an error."""
import argparse
import sys

from .generator import generate_files


def main(argv=None):
    ap = argparse.ArgumentParser(description="CompLL: gradient-compression DSL -> sm_100a CUDA (and CPU C++)")
    ap.add_argument("input_file", help="DSL source (.pse)")
    ap.add_argument("-b", "--body", action="store_true", help="generate the kernels")
    ap.add_argument("-w", "--wrapper", action="store_true", help="generate the C launcher")
    ap.add_argument("-r", "--register", action="store_true", help="generate the framework binding")
    ap.add_argument("-f", "--framework", default="torch", help="target framework (torch)")
    ap.add_argument("-t", "--target", default="all", choices=["cuda", "cpu", "all"],
                    help="sm_100a kernels, sequential C++, or both (default)")
    ap.add_argument("-o", "--output", default="output", help="output directory")
    ap.add_argument("--build", action="store_true", help="also compile the result (nvcc / g++)")
    a = ap.parse_args(argv)
    if not (a.body or a.wrapper or a.register):
        a.body = a.wrapper = a.register = True
    files = generate_files(a.input_file, a.output, body=a.body, wrapper=a.wrapper,
                           register=a.register, framework=a.framework, build=a.build,
                           target=a.target)
    for f in files:
        print(f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
