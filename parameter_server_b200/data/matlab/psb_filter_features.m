function [X, keep, group_offset] = psb_filter_features(X, min_count, group_offset)
% PSB_FILTER_FEATURES  Drop the columns of X that occur in at most min_count rows (tail features).
%   [X, keep] = psb_filter_features(X, 4)
%   [X, keep, group_offset] = psb_filter_features(X, 4, group_offset)
%       group_offset(g) is the first column (1-based) of feature group g, with one entry past the last group;
%       the returned offsets describe the same groups in the filtered matrix.
% Same job as the solver's tail_feature_freq filter, and as the reference's filter_fea.m script.
  keep = full(sum(X ~= 0, 1)) > min_count;
  if nargin >= 3 && ~isempty(group_offset)
    kept_before = [0, cumsum(keep)];                              % kept columns among the first c columns
    group_offset = kept_before(group_offset) + 1;
  else
    group_offset = [];
  end
  X = X(:, keep);
end
