"""`python main.py ...`: the command line, as in the reference's main.py. See
llm_infer_engine_b200/cli/main.py for the options."""
import sys

from llm_infer_engine_b200.cli.main import main

if __name__ == "__main__":
    sys.exit(main())
