// Episode dataset reader (host only): see dataset_host.cpp.
#pragma once

#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/bpsn.h"

namespace bpsn {

struct DatasetScene {
  std::string sceneId;      // as written in the episode file, e.g. "gibson/Allensville.glb"
  std::string navmeshPath;  // asset_path / scene id with the extension replaced by ".navmesh"
  std::vector<bpsn_episode> episodes;
};

// Reads every *.json.gz under datasetPath (file-name order, empty files skipped) with up to
// numThreads threads.  Returns false and sets *err on the first problem.
bool loadDataset(const std::string& datasetPath, const std::string& assetPath, uint32_t numThreads,
                 std::vector<DatasetScene>* out, std::string* err);

}  // namespace bpsn
