# Common entry points; every target is a thin wrapper around a command documented in README.md.
PYTHON ?= python
NPROC  ?= 1

.PHONY: build test test-gpu bench estimate clean

build:            ## compile pithtrain_b200/csrc/*.cu for sm_100a into pithtrain_b200/_lib/libpithb200.so
	$(PYTHON) -m pithtrain_b200.build

test: build       ## CPU tier (unit tests and 2-4 rank gloo jobs)
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: build   ## GPU tier, on a B200
	$(PYTHON) -m pytest tests -q -m gpu

bench: build      ## headline benchmark; NPROC=8 runs the pp2 x ep4 mesh through torchrun
ifeq ($(NPROC),1)
	$(PYTHON) bench.py --gpus 1
else
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus $(NPROC)
endif

estimate:         ## memory estimate of the headline 8-GPU job
	$(PYTHON) -m pithtrain_b200.tools.memory_estimator --model examples/pretrain_lm/qwen3-30b-a3b/config.json \
	    --pp-size 2 --ep-size 4 --global-batch-size 256 --sequence-length 4096 --detail

clean:
	rm -rf pithtrain_b200/_lib/obj
