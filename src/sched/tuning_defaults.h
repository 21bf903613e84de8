// Selection table measured on 8 x B200 (NVLink 5 through NVSwitch) with nccl_b200/utils/tune.py:
// rows are [largest message in bytes (nccl-tests size convention), variant, CTAs].
#pragma once
namespace b200 {
static const char kDefaultTuningJson[] = R"JSON({
"2": {
 "all_reduce": [[1048576,"LL",0],[4194304,"NVLS",128],[1099511627776,"P2P",128]],
 "all_gather": [[1048576,"LL",0],[4194304,"MC",8],[1099511627776,"PUSH",128]],
 "reduce_scatter": [[1048576,"LL",0],[4194304,"NVLS",128],[1099511627776,"P2P",128]],
 "all_to_all": [[1048576,"LL",0],[4194304,"PUSH",64],[1099511627776,"PUSH",128]],
 "broadcast": [[1048576,"LL",0],[4194304,"MC",16],[16777216,"PULL",64],[67108864,"MC",16],[268435456,"PULL",64],[1099511627776,"PUSH",128]]
},
"3": {
 "all_reduce": [[524288,"LL",0],[4194304,"NVLS",64],[268435456,"NVLS",16],[1099511627776,"NVLS",64]],
 "all_gather": [[1048576,"LL",0],[4194304,"MC",128],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "reduce_scatter": [[4194304,"LL",0],[16777216,"NVLS",16],[1099511627776,"P2P",128]],
 "all_to_all": [[4194304,"LL",0],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "broadcast": [[262144,"LL",0],[1048576,"MC",16],[16777216,"MC",128],[268435456,"MC",16],[1099511627776,"MC",64]]
},
"4": {
 "all_reduce": [[524288,"LL",0],[4194304,"NVLS",64],[268435456,"NVLS",16],[1099511627776,"NVLS",64]],
 "all_gather": [[1048576,"LL",0],[4194304,"MC",128],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "reduce_scatter": [[4194304,"LL",0],[16777216,"NVLS",16],[1099511627776,"P2P",128]],
 "all_to_all": [[4194304,"LL",0],[16777216,"PUSH",64],[1099511627776,"PUSH",128]],
 "broadcast": [[262144,"LL",0],[1048576,"MC",16],[16777216,"MC",128],[268435456,"MC",16],[1099511627776,"MC",64]]
}
})JSON";
}  // namespace b200
