// mgpu::sharded_segreduce: one array reduced by segment across several GPUs
// (or across several calls on one GPU). No counterpart in the reference.
#pragma once
#include "b200/shard.hxx"
