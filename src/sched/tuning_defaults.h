// Selection table measured on 8 x B200 (NVLink 5 through NVSwitch) with nccl_b200/utils/tune.py:
// rows are [largest message in bytes (nccl-tests size convention), variant, CTAs].
#pragma once
namespace b200 {
static const char kDefaultTuningJson[] = R"JSON({
"2": {
 "all_reduce": [[262144,"LL",0],[4194304,"NVLS",8],[1099511627776,"P2P",128]],
 "all_gather": [[524288,"LL",0],[4194304,"MC",8],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "reduce_scatter": [[524288,"LL",0],[4194304,"NVLS",8],[1099511627776,"P2P",128]],
 "all_to_all": [[524288,"LL",0],[4194304,"PUSH",8],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "broadcast": [[262144,"LL",0],[1048576,"MC",8],[1099511627776,"PULL",64]]
}
})JSON";
}  // namespace b200
