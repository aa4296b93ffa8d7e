"""Multi-node speed test: test/test.py under ``torchrun --nnodes`` (the
rendezvous comes from the environment; reference: test/test_multinode.py)."""
import importlib.util, os
_spec = importlib.util.spec_from_file_location("_fo_speed_test", os.path.join(os.path.dirname(os.path.abspath(__file__)), "test.py"))
speed_test = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(speed_test)

if __name__ == "__main__":
    speed_test.main()
