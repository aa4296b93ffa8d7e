"""Multi-node speed test: test/test.py under ``torchrun --nnodes`` (the
rendezvous comes from the environment; reference: test/test_multinode.py)."""
import test as speed_test

if __name__ == "__main__":
    speed_test.main()
